// Decode attention over an UNQUANTISED (fp16 / bf16) paged KV cache with grouped query heads.
//
// K_pages / V_pages [num_pages, page_size, Hkv, D], block_table [B, max_blocks], lengths [B], q [B, Hq, D]:
// out[b, hq] = softmax(scale * q . K[b, :len_b, hq / group]) V[b, :len_b, hq / group], scores and sums in fp32.
// The cache is four (q4: eight) times the bytes of the quantised one, so the kernel is a plain HBM streamer:
// grid (splits, Hkv, B); a warp takes four tokens per pass, eight lanes per token, each lane 16 consecutive
// dimensions of the K and of the V row (two 16-byte loads each) and the running softmax state of up to four query
// heads of the group; lanes, warps and finally the splits are merged with the usual (max, sum, weighted rows) rule.
#include "common.cuh"

#include <algorithm>

namespace b200q {

namespace {

constexpr int kWarps = 4;
constexpr int kHeadChunk = 4;       // query heads of a group handled per pass over the tokens
constexpr int kPartStride = 130;    // floats per partial: max, sum, 128 weighted dims

struct Fp16AttnParams {
    const void* q; const void* k_pages; const void* v_pages; const int32_t* block_table; const int32_t* lengths;
    void* out; float* workspace;
    int B, Hq, Hkv, D, P, max_blocks, splits, dtype;
    int64_t num_pages;
    float scale;
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 16 consecutive elements of a row starting at dimension d0 (zero beyond D); `vec` when D is a multiple of 8 and
// the row base is 16-byte aligned.
template <typename T>
__device__ __forceinline__ void load16(float (&dst)[16], const T* row, int d0, int D, bool vec) {
    if (vec) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int d = d0 + 8 * h;
            if (d < D) {
                const uint4 u = *reinterpret_cast<const uint4*>(row + d);
                const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
                for (int i = 0; i < 8; ++i) dst[8 * h + i] = to_f32<T>(e[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) dst[8 * h + i] = 0.0f;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = d0 + i < D ? to_f32<T>(row[d0 + i]) : 0.0f;
    }
}

__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// (max, sum, weighted rows) of two disjoint token sets -> of their union; the maxima are in log2 units
__device__ __forceinline__ void merge_state(float& m, float& l, float (&acc)[16], float m_o, float l_o, const float (&acc_o)[16]) {
    const float M = fmaxf(m, m_o);
    const float a = m == -INFINITY ? 0.0f : exp2_fast(m - M);
    const float b = m_o == -INFINITY ? 0.0f : exp2_fast(m_o - M);
    l = l * a + l_o * b;
#pragma unroll
    for (int e = 0; e < 16; ++e) acc[e] = acc[e] * a + acc_o[e] * b;
    m = M;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) paged_fp16_attn_kernel(const __grid_constant__ Fp16AttnParams p) {
    __shared__ float part[kWarps][kHeadChunk][kPartStride];
    const int s = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tg = lane >> 3, sl = lane & 7, d0 = 16 * sl;
    const int group = p.Hq / p.Hkv;
    const int cap = p.max_blocks * p.P;
    const int L = min(max(p.lengths[b], 0), cap);
    const int npages = (L + p.P - 1) / p.P;
    const int per = (npages + p.splits - 1) / p.splits;
    const int lo = min(L, s * per * p.P), hi = min(L, (s + 1) * per * p.P);
    const T* kp = reinterpret_cast<const T*>(p.k_pages);
    const T* vp = reinterpret_cast<const T*>(p.v_pages);
    const bool vec = (p.D % 8 == 0) && ((reinterpret_cast<uintptr_t>(kp) | reinterpret_cast<uintptr_t>(vp) |
                                         reinterpret_cast<uintptr_t>(p.q)) % 16 == 0);
    const int32_t* bt = p.block_table + (size_t)b * p.max_blocks;
    const uint32_t tmask = 0xFFu << (8 * tg);
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int pshift = (p.P & (p.P - 1)) == 0 ? 31 - __clz(p.P) : -1;     // page size a power of two: shifts, no division

    for (int c0 = 0; c0 < group; c0 += kHeadChunk) {
        const int nh = min(kHeadChunk, group - c0);
        float qf[kHeadChunk][16], acc[kHeadChunk][16], m[kHeadChunk], l[kHeadChunk];
#pragma unroll
        for (int i = 0; i < kHeadChunk; ++i) {
            m[i] = -INFINITY;
            l[i] = 0.0f;
#pragma unroll
            for (int e = 0; e < 16; ++e) acc[i][e] = 0.0f;
            if (i < nh) {
                const T* qrow = reinterpret_cast<const T*>(p.q) + ((size_t)b * p.Hq + (size_t)h * group + c0 + i) * p.D;
                load16<T>(qf[i], qrow, d0, p.D, vec);
            } else {
#pragma unroll
                for (int e = 0; e < 16; ++e) qf[i][e] = 0.0f;
            }
        }
#pragma unroll 2
        for (int j = lo + warp * 4 + tg; j < hi; j += kWarps * 4) {
            const int blk = pshift >= 0 ? j >> pshift : j / p.P;
            const int page = bt[blk];
            if (page < 0 || page >= p.num_pages) continue;            // unassigned page: its tokens take no part
            const size_t row = (((size_t)page * p.P + (j - blk * p.P)) * p.Hkv + h) * p.D;
            float kf[16], vf[16];
            load16<T>(kf, kp + row, d0, p.D, vec);
            load16<T>(vf, vp + row, d0, p.D, vec);
#pragma unroll
            for (int i = 0; i < kHeadChunk; ++i) {
                if (i >= nh) break;
                float dot = 0.0f;
#pragma unroll
                for (int e = 0; e < 16; ++e) dot = fmaf(qf[i][e], kf[e], dot);
                dot += __shfl_xor_sync(tmask, dot, 1);        // the eight lanes of this token only: the other token
                dot += __shfl_xor_sync(tmask, dot, 2);        // groups of the warp may have left the loop
                dot += __shfl_xor_sync(tmask, dot, 4);
                const float sc = dot * scale_log2;            // scores in log2 units: one ex2 per exponential
                const float m_new = fmaxf(m[i], sc);
                const float alpha = exp2_fast(m[i] - m_new);  // ex2(-inf) = 0 for the first token
                const float beta = exp2_fast(sc - m_new);
                l[i] = l[i] * alpha + beta;
                m[i] = m_new;
#pragma unroll
                for (int e = 0; e < 16; ++e) acc[i][e] = acc[i][e] * alpha + beta * vf[e];
            }
        }
        // the four token lanes of a warp (xor 8, 16), then the warps through shared memory
#pragma unroll
        for (int i = 0; i < kHeadChunk; ++i) {
#pragma unroll
            for (int o = 8; o <= 16; o <<= 1) {
                const float m_o = __shfl_xor_sync(0xffffffffu, m[i], o);
                const float l_o = __shfl_xor_sync(0xffffffffu, l[i], o);
                float acc_o[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) acc_o[e] = __shfl_xor_sync(0xffffffffu, acc[i][e], o);
                merge_state(m[i], l[i], acc[i], m_o, l_o, acc_o);
            }
            if (tg == 0) {
                if (sl == 0) { part[warp][i][0] = m[i]; part[warp][i][1] = l[i]; }
#pragma unroll
                for (int e = 0; e < 16; ++e) part[warp][i][2 + d0 + e] = acc[i][e];
            }
        }
        __syncthreads();
        // thread d merges the warps' rows of dimension d, head by head
        const int d = threadIdx.x;
        for (int i = 0; i < nh; ++i) {
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) M = fmaxf(M, part[w][i][0]);
            float lsum = 0.0f, o = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float mw = part[w][i][0];
                const float f = mw == -INFINITY ? 0.0f : exp2_fast(mw - M);
                lsum += part[w][i][1] * f;
                o += part[w][i][2 + d] * f;
            }
            const int hq = h * group + c0 + i;
            if (p.splits == 1) {
                if (d < p.D)
                    reinterpret_cast<T*>(p.out)[((size_t)b * p.Hq + hq) * p.D + d] = from_f32<T>(lsum > 0.0f ? o / lsum : 0.0f);
            } else {
                float* dst = p.workspace + (((size_t)s * p.B + b) * p.Hq + hq) * kPartStride;
                if (d == 0) { dst[0] = M; dst[1] = lsum; }
                if (d < p.D) dst[2 + d] = o;
            }
        }
        __syncthreads();
    }
}

template <typename T>
__global__ void __launch_bounds__(128) paged_fp16_merge_kernel(const __grid_constant__ Fp16AttnParams p) {
    const int item = blockIdx.x;                  // b * Hq + hq
    const int d = threadIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < p.splits; ++s) M = fmaxf(M, p.workspace[((size_t)s * p.B * p.Hq + item) * kPartStride]);
    float lsum = 0.0f, o = 0.0f;
    for (int s = 0; s < p.splits; ++s) {
        const float* src = p.workspace + ((size_t)s * p.B * p.Hq + item) * kPartStride;
        const float f = src[0] == -INFINITY ? 0.0f : exp2f(src[0] - M);      // the maxima are in log2 units
        lsum += src[1] * f;
        if (d < p.D) o += src[2 + d] * f;
    }
    if (d < p.D) reinterpret_cast<T*>(p.out)[(size_t)item * p.D + d] = from_f32<T>(lsum > 0.0f ? o / lsum : 0.0f);
}

int splits_for(int B, int Hkv, int max_blocks) {
    const int want = (4 * sm_count() + B * Hkv - 1) / (B * Hkv);
    return std::max(1, std::min({want, 64, max_blocks}));
}

}  // namespace

size_t paged_fp16_workspace_bytes_impl(int B, int Hq, int Hkv, int max_blocks) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || max_blocks <= 0) return 0;
    const int s = splits_for(B, Hkv, max_blocks);
    return s == 1 ? 0 : (size_t)s * B * Hq * kPartStride * sizeof(float);
}

int paged_fp16_gqa_decode_impl(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_table,
                               const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes, int B, int Hq,
                               int Hkv, int D, int page_size, int64_t num_pages, int max_blocks, float scale, int dtype,
                               cudaStream_t stream) {
    if (q == nullptr || k_pages == nullptr || v_pages == nullptr || block_table == nullptr || lengths == nullptr ||
        out == nullptr)
        return B200Q_ERR_BAD_ARG;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || D <= 0 || page_size <= 0 || num_pages <= 0 || max_blocks <= 0)
        return B200Q_ERR_BAD_ARG;
    if (D > 128 || (dtype != B200Q_F16 && dtype != B200Q_BF16) || Hkv > 65535 || B > 65535) return B200Q_ERR_UNSUPPORTED;
    Fp16AttnParams p = {};
    p.q = q; p.k_pages = k_pages; p.v_pages = v_pages; p.block_table = block_table; p.lengths = lengths; p.out = out;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.P = page_size; p.max_blocks = max_blocks; p.dtype = dtype;
    p.num_pages = num_pages; p.scale = scale;
    p.splits = splits_for(B, Hkv, max_blocks);
    if (p.splits > 1) {
        const size_t need = paged_fp16_workspace_bytes_impl(B, Hq, Hkv, max_blocks);
        if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0)
            return B200Q_ERR_WORKSPACE;
        p.workspace = reinterpret_cast<float*>(workspace);
    }
    const dim3 grid(p.splits, Hkv, B);
    if (dtype == B200Q_F16) paged_fp16_attn_kernel<__half><<<grid, kWarps * 32, 0, stream>>>(p);
    else paged_fp16_attn_kernel<__nv_bfloat16><<<grid, kWarps * 32, 0, stream>>>(p);
    int rc = finish_launch();
    if (rc != B200Q_OK || p.splits == 1) return rc;
    if (dtype == B200Q_F16) paged_fp16_merge_kernel<__half><<<B * Hq, 128, 0, stream>>>(p);
    else paged_fp16_merge_kernel<__nv_bfloat16><<<B * Hq, 128, 0, stream>>>(p);
    return finish_launch();
}

}  // namespace b200q
