// Decode-layer glue between the matvec and attention kernels: split the fused QKV row, apply the
// interleaved-pair rotary embedding to q and k, and append the new token's k / v - quantised with
// the cache's own rule - to its page.
//
//   q_out[b, h, :]  = rope(qkv[b, h*D : (h+1)*D], pos[b])                          h < Hq
//   k = rope(qkv[b, (Hq + h)*D ...], pos[b]) ; v = qkv[b, (Hq + Hkv + h)*D ...]    h < Hkv
//   page = block_table[b, pos[b] / P], slot = pos[b] % P
//   per group of G along D: scale = max(max|v|, 1e-8) / (127 | 7) (fp32, stored fp16),
//                           code = clip(rint(v / scale), -127|-7, 127|7) + (128 | 8)
//
// RoPE follows the reference (ops/rope_ops.py:61-75): pairs (2i, 2i+1), cos/sin tables [S, D/2]
// in fp32, y_even = x_even*cos - x_odd*sin, y_odd = x_even*sin + x_odd*cos, rounded to fp16.
// The quantisation rule is _quantize_group_symmetric_8 / _4 of the reference cache
// (ops/paged_quantized_kv_ops.py:146-175); the reference itself has no append kernel (its update
// kernels copy the whole cache per token).
//
// One warp per (sequence, head); head_dim <= 128 and even; lanes own 4 consecutive elements.
#include "common.cuh"

#include <algorithm>

namespace b200q {

B200Q_DEFINE_STATUS_WORD(stack_read_status)

namespace {

struct RopeAppendParams {
    const __half* qkv;          // [B, (Hq + 2 Hkv) * D]
    const float* cos_table;     // [S, D/2]
    const float* sin_table;
    const int32_t* positions;   // [B]
    const int32_t* block_table; // [B, max_blocks]
    __half* q_out;              // [B, Hq, D]
    uint8_t* k_codes; uint8_t* v_codes;   // [num_pages, P, Hkv, D or D/2]
    __half* k_scales; __half* v_scales;   // [num_pages, P, Hkv, Gd]
    int B, Hq, Hkv, D, P, max_blocks, G, Gd, bits, table_len;
    int64_t num_pages;
};

__global__ void __launch_bounds__(128) rope_kv_append_kernel(const __grid_constant__ RopeAppendParams p) {
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int heads = p.Hq + 2 * p.Hkv;
    pdl_launch_dependents();
    pdl_wait();
    if (item >= p.B * heads) return;
    const int b = item / heads;
    const int hh = item - b * heads;
    const int pos = p.positions[b];
    const int d0 = lane * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const bool live = d0 < p.D;
    if (live) {
        const uint2 u = *reinterpret_cast<const uint2*>(p.qkv + ((size_t)b * heads + hh) * p.D + d0);
        const __half2 h0 = *reinterpret_cast<const __half2*>(&u.x), h1 = *reinterpret_cast<const __half2*>(&u.y);
        v[0] = __low2float(h0); v[1] = __high2float(h0); v[2] = __low2float(h1); v[3] = __high2float(h1);
    }
    const bool is_v = hh >= p.Hq + p.Hkv;
    // a position outside the rotary table: the row passes through unrotated and the event is recorded
    if (!is_v && lane == 0 && (pos < 0 || pos >= p.table_len)) atomicMax(&g_device_status, (int)EV_ROPE_POSITION);
    if (!is_v && live && pos >= 0 && pos < p.table_len) {
        const int half_d = p.D / 2;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float c = p.cos_table[(size_t)pos * half_d + d0 / 2 + i];
            const float s = p.sin_table[(size_t)pos * half_d + d0 / 2 + i];
            const float xe = v[2 * i], xo = v[2 * i + 1];
            // two separately rounded products and one sum, as the reference's elementwise expression
            v[2 * i] = __fsub_rn(__fmul_rn(xe, c), __fmul_rn(xo, s));
            v[2 * i + 1] = __fadd_rn(__fmul_rn(xe, s), __fmul_rn(xo, c));
        }
    }
    // values as the cache / attention see them: rounded to fp16
    __half hv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { hv[i] = __float2half_rn(v[i]); v[i] = __half2float(hv[i]); }

    if (hh < p.Hq) {
        if (live) {
            uint2 o;
            o.x = (uint32_t)__half_as_ushort(hv[0]) | ((uint32_t)__half_as_ushort(hv[1]) << 16);
            o.y = (uint32_t)__half_as_ushort(hv[2]) | ((uint32_t)__half_as_ushort(hv[3]) << 16);
            *reinterpret_cast<uint2*>(p.q_out + ((size_t)b * p.Hq + hh) * p.D + d0) = o;
        }
        return;
    }
    // ---- k or v: quantise this head's row into its page slot ----
    const int hkv = is_v ? hh - p.Hq - p.Hkv : hh - p.Hq;
    const int blk = pos / p.P;
    int page = (pos >= 0 && blk < p.max_blocks) ? p.block_table[(size_t)b * p.max_blocks + blk] : -1;
    if (page < 0 || page >= p.num_pages) {                // unassigned page: nothing is written, the event is recorded
        if (lane == 0) atomicMax(&g_device_status, (int)EV_KV_PAGE_UNASSIGNED);
        return;
    }
    const int slot = pos % p.P;
    // group max over G elements = G/4 consecutive lanes (G a multiple of 4, power of two <= 128)
    float mx = live ? fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))) : 0.0f;
    const int lanes_per_group = p.G / 4;
    for (int o = 1; o < lanes_per_group; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float limit = p.bits == 8 ? 127.0f : 7.0f;
    const float offset = p.bits == 8 ? 128.0f : 8.0f;
    const float scale = __fdiv_rn(fmaxf(mx, 1e-8f), limit);
    uint32_t codes[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float qv = fminf(fmaxf(rintf(__fdiv_rn(v[i], scale)), -limit), limit) + offset;
        codes[i] = (uint32_t)(int)qv;
    }
    const size_t tok = ((size_t)page * p.P + slot) * p.Hkv + hkv;
    uint8_t* cdst = is_v ? p.v_codes : p.k_codes;
    __half* sdst = is_v ? p.v_scales : p.k_scales;
    if (live) {
        if (p.bits == 8) {
            const uint32_t w = codes[0] | (codes[1] << 8) | (codes[2] << 16) | (codes[3] << 24);
            *reinterpret_cast<uint32_t*>(cdst + tok * p.D + d0) = w;
        } else {
            const uint16_t w = (uint16_t)(codes[0] | (codes[1] << 4) | (codes[2] << 8) | (codes[3] << 12));
            *reinterpret_cast<uint16_t*>(cdst + tok * (p.D / 2) + d0 / 2) = w;
        }
        if ((lane % lanes_per_group) == 0) sdst[tok * p.Gd + d0 / p.G] = __float2half_rn(scale);
    }
}

// Symmetric group-wise quantisation of [rows, D] values with the cache rule above: one thread per (row, group)
// (per row when the group size is odd, so that a packed byte never straddles two threads).
template <typename T>
__global__ void __launch_bounds__(256) quantize_kv_kernel(const T* __restrict__ values, uint8_t* __restrict__ codes,
                                                          __half* __restrict__ scales, int64_t rows, int D, int G, int Gd,
                                                          int bits, bool per_row) {
    const int64_t items = per_row ? rows : rows * Gd;
    const float limit = bits == 8 ? 127.0f : 7.0f;
    const float offset = bits == 8 ? 128.0f : 8.0f;
    const int dp = bits == 4 ? (D + 1) / 2 : D;
    for (int64_t it = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; it < items; it += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = per_row ? it : it / Gd;
        const int g_lo = per_row ? 0 : (int)(it - row * Gd);
        const int g_hi = per_row ? Gd : g_lo + 1;
        const T* src = values + row * D;
        uint8_t* dst = codes + row * dp;
        for (int g = g_lo; g < g_hi; ++g) {
            const int d_lo = g * G, d_hi = min(D, d_lo + G);
            float mx = 0.0f;
            for (int d = d_lo; d < d_hi; ++d) mx = fmaxf(mx, fabsf(to_f32(src[d])));
            const float scale = __fdiv_rn(fmaxf(mx, 1e-8f), limit);
            scales[row * Gd + g] = __float2half_rn(scale);
            for (int d = d_lo; d < d_hi; ++d) {
                const float qv = fminf(fmaxf(rintf(__fdiv_rn(to_f32(src[d]), scale)), -limit), limit) + offset;
                const uint32_t c = (uint32_t)(int)qv;
                if (bits == 8) {
                    dst[d] = (uint8_t)c;
                } else if (d & 1) {
                    dst[d >> 1] = (uint8_t)(dst[d >> 1] | (c << 4));     // the low nibble was written just before by this thread
                } else {
                    dst[d >> 1] = (uint8_t)c;                            // high nibble zero (stays zero for an odd D)
                }
            }
        }
    }
}

}  // namespace

int quantize_kv_impl(int bits, const void* values, uint8_t* codes, void* scales, int64_t rows, int D, int group_size,
                     int in_dtype, cudaStream_t stream) {
    if ((bits != 4 && bits != 8) || values == nullptr || codes == nullptr || scales == nullptr) return B200Q_ERR_BAD_ARG;
    if (rows <= 0 || D <= 0 || group_size <= 0 || !is_act_dtype(in_dtype)) return B200Q_ERR_BAD_ARG;
    const int Gd = (D + group_size - 1) / group_size;
    const bool per_row = bits == 4 && (group_size & 1);
    const int64_t items = per_row ? rows : rows * Gd;
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((items + 255) / 256, (int64_t)sm_count() * 16));
    if (in_dtype == B200Q_F16)
        quantize_kv_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)values, codes, (__half*)scales, rows, D, group_size,
                                                            Gd, bits, per_row);
    else
        quantize_kv_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)values, codes, (__half*)scales, rows,
                                                                   D, group_size, Gd, bits, per_row);
    return finish_launch();
}

int rope_kv_append_impl(const void* qkv, const float* cos_table, const float* sin_table, const int32_t* positions,
                        const int32_t* block_table, void* q_out, uint8_t* k_codes, uint8_t* v_codes, void* k_scales,
                        void* v_scales, int bits, int B, int Hq, int Hkv, int D, int page_size, int64_t num_pages,
                        int max_blocks, int group_size, int table_len, cudaStream_t stream) {
    if (qkv == nullptr || cos_table == nullptr || sin_table == nullptr || positions == nullptr || block_table == nullptr ||
        q_out == nullptr || k_codes == nullptr || v_codes == nullptr || k_scales == nullptr || v_scales == nullptr)
        return B200Q_ERR_BAD_ARG;
    if ((bits != 4 && bits != 8) || B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || page_size <= 0 || num_pages <= 0 ||
        max_blocks <= 0 || group_size <= 0 || table_len <= 0)
        return B200Q_ERR_BAD_ARG;
    if (D > 128 || D % 4 != 0 || group_size % 4 != 0 || (group_size & (group_size - 1)) != 0 || group_size > 128 ||
        D % group_size != 0)
        return B200Q_ERR_UNSUPPORTED;
    RopeAppendParams p = {};
    p.qkv = (const __half*)qkv; p.cos_table = cos_table; p.sin_table = sin_table; p.positions = positions;
    p.block_table = block_table; p.q_out = (__half*)q_out; p.k_codes = k_codes; p.v_codes = v_codes;
    p.k_scales = (__half*)k_scales; p.v_scales = (__half*)v_scales;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.P = page_size; p.max_blocks = max_blocks; p.G = group_size;
    p.Gd = D / group_size; p.bits = bits; p.table_len = table_len; p.num_pages = num_pages;
    const int warps = 4;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((B * (Hq + 2 * Hkv) + warps - 1) / warps);
    cfg.blockDim = dim3(warps * 32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning_get("no_pdl") ? 0 : 1;
    if (cudaLaunchKernelEx(&cfg, rope_kv_append_kernel, p) != cudaSuccess) return B200Q_ERR_LAUNCH;
    return finish_launch();
}

}  // namespace b200q
