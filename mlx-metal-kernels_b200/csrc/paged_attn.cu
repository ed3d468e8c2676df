// Paged quantized-KV GQA decode attention (q4 / q8 symmetric, fp16 scales) for sm_100a.
//
//   out[b, hq] = softmax_j( scale * q[b, hq] . Khat[j, hkv] ) . Vhat[j, hkv],  hkv = hq / (Hq/Hkv)
//   Khat = fp16((code - 8|128) * |k_scale|)   over the valid tokens j of sequence b.
//
// Fast kernel (head_dim 128, page size 16, q in fp16, fp16 scales, group size 32 or 64, at most 8
// query heads per kv head, at most 8 kv heads):
//   * the (sequence, page) pairs of the whole batch form one flattened list that is cut into
//     equal contiguous ranges, one per CTA ("stream-K" over ragged lengths: every CTA streams the
//     same number of pages whatever the length distribution).  A CTA writes one partial
//     (max, sum, accumulator) per sequence it touches; a second small kernel merges them.
//   * warp w of a CTA owns kv head w % Hkv (and, when there are fewer than 8 kv heads, every
//     (8/Hkv)-th page of the range).  It is self-contained: it looks up its page ids 32 at a time,
//     and every lane copies exactly the bytes IT will consume (16 bytes of two K token rows,
//     8 bytes of four V token rows) with cp.async into a private ring in shared memory, several
//     pages ahead.  No CTA-wide barrier, no bank conflicts (the ring is laid out [piece][lane]).
//     Measured on B200: the bulk-copy (TMA) engine needs >= 2 KB per copy to reach HBM speed,
//     and a token row of one page is 512 B, so per-lane asynchronous copies are the faster route.
//   * scores S[token, head] = K Q^T on mma.sync.m16n8k16 with the 16 tokens of a page as rows (in-register
//     dequantised K is the A operand) and the up to 8 query heads of the group as columns: no padding rows and
//     no zero operand registers.  Online softmax in fp32 (a lane holds two heads of tokens g and g + 8; the row
//     maximum is a butterfly over the 8 token lanes, the sums stay per lane until a partial is written).  One
//     movmatrix per 8 tokens turns the probabilities into the B operand of O^T[d, head] += V^T P, where V^T is
//     the A operand built from the four token rows with one byte-permute per word pair.  KV bytes are read once
//     per kv head, not once per query head; Khat / Vhat are bit-identical to the reference's fp16 dequantised
//     cache.
//
// Everything else (other head dims, bf16 queries, other group sizes) runs the simple kernel: one
// warp per (sequence, query head), the reference's streaming-softmax loop.
#include "common.cuh"

#include <algorithm>
#include <cmath>
#include <mutex>

namespace b200q {

B200Q_DEFINE_STATUS_WORD(attn_read_status)

namespace {

constexpr int kAttnWarps = 8;
constexpr int kAttnThreads = kAttnWarps * 32;
#ifndef B200Q_ATTN_CTAS
#define B200Q_ATTN_CTAS 2                    // resident CTAs per SM of the fast kernel's dense shape
#endif
constexpr int kMaxGrid = 152 * B200Q_ATTN_CTAS;   // upper bound on CTAs of the fast kernel (sizes the workspace)
constexpr int kMaxBatchFast = 2048;       // prefix sums of page counts live in shared memory
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
    const __half* q;            // [B, Hq, D]
    const uint8_t* k_codes;
    const uint8_t* v_codes;
    const __half* k_scales;
    const __half* v_scales;
    const int32_t* block_table; // [B, max_blocks]
    const int32_t* lengths;     // [B]
    float* partial;             // [grid + B][Hq][D + 2]  (acc[D], max, sum); slot = range + sequence
    void* out;                  // [B, Hq, D]
    int B, Hq, Hkv, D, P, max_blocks, G, Gd, group;
    int64_t num_pages;
    float scale;
    int q_dtype;
    int bits;
    int stages;                 // pages in flight per warp
    int subs;                   // ranges per CTA (8 / Hkv)
    int row_bytes;              // bytes of one token row of codes, all kv heads
    int scale_row_halves;       // halves of one token row of scales, all kv heads
    uint32_t off_prefix, off_ring, slot_bytes;
    int grid;
    int sink, window;           // window > 0: only positions < sink or >= length - window are attended
    TpOut tp_out;               // tensor-parallel exchange of the merged rows (world == 0: off)
};

__device__ __forceinline__ int clamp_len(int len, int cap) { return max(0, min(len, cap)); }

// Pages of one sequence that hold at least one attended position.  Dense: all of them.  With a window: the
// pages of the sink tokens that lie below the window, then the pages from the window's first position on.
struct SeqPages { int n, sink_pages, first_recent, L; };
__device__ __forceinline__ SeqPages seq_pages(int len, int cap, int P, int sink, int window) {
    const int L = clamp_len(len, cap);
    const int n_all = (L + P - 1) / P;
    if (window <= 0 || L <= 0) return {n_all, n_all, n_all, L};
    const int lo = max(0, L - window);
    const int sink_pages = (min(sink, lo) + P - 1) / P;
    const int first_recent = max(sink_pages, lo / P);
    return {sink_pages + n_all - first_recent, sink_pages, first_recent, L};
}
// bit t set: slot t of page pg (16 slots) is an attended position of a sequence of L tokens
__device__ __forceinline__ uint32_t page_mask16(int pg, int L, int sink, int window) {
    const int valid = min(16, L - pg * 16);
    uint32_t m = valid >= 16 ? 0xFFFFu : ((1u << max(valid, 0)) - 1u);
    if (window > 0) {
        const int lo_t = max(0, L - window) - pg * 16;      // first slot of the window in this page
        const int sink_t = sink - pg * 16;                    // slots below this are sink tokens
        const uint32_t recent = lo_t <= 0 ? 0xFFFFu : (lo_t >= 16 ? 0u : (0xFFFFu << lo_t) & 0xFFFFu);
        const uint32_t sinks = sink_t <= 0 ? 0u : (sink_t >= 16 ? 0xFFFFu : (1u << sink_t) - 1u);
        m &= recent | sinks;
    }
    return m;
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_8(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Prefix sums of per-sequence page counts into shared memory; returns the total.
__device__ int build_prefix(const AttnParams& p, int* prefix) {
    // executed by every thread of the CTA up to the final __syncthreads
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int running = 0;
        for (int b0 = 0; b0 < p.B; b0 += 32) {
            const int b = b0 + lane;
            int n = 0;
            if (b < p.B) n = seq_pages(p.lengths[b], p.max_blocks * p.P, p.P, p.sink, p.window).n;
            int incl = n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (b < p.B) prefix[b] = running + incl - n;
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) prefix[p.B] = running;
    }
    __syncthreads();
    return prefix[p.B];
}

// largest b with prefix[b] <= f (f < prefix[B])
__device__ __forceinline__ int find_sequence(const int* prefix, int B, int f) {
    int lo = 0, hi = B - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (prefix[mid] <= f) lo = mid; else hi = mid - 1;
    }
    return lo;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ------------------------------------------------------------------------------------------------
// Per-warp building blocks shared by the split-KV kernel and the cluster kernel: a warp owns one kv head and
// walks pages of it; every lane copies exactly the bytes IT will consume into a private ring slot.
// ------------------------------------------------------------------------------------------------
struct WarpAcc {
    uint32_t qb[8][2];          // Q^T as B operand: [mma][b0b1, b2b3], column g = query head g of the group
    float o[8][4];              // O^T tiles: rows d, cols heads
    float m_run[2];             // running max of query heads 2t, 2t+1 of the group
    float l_run[2];             // this lane's share (tokens g, g + 8 of every page) of their running sums
};
__device__ __forceinline__ void acc_reset(WarpAcc& a) {
    a.m_run[0] = a.m_run[1] = -INFINITY;
    a.l_run[0] = a.l_run[1] = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) a.o[i][e] = 0.0f;
}
// Q fragments of one kv head's group: row r of `qrows` (D halves apart) is query head r of the group (r < group <= 8).
// qrows may point to global or shared memory.
template <int BITS>
__device__ __forceinline__ void load_q_frags(WarpAcc& a, const __half* qrows, int group, int g, int t) {
    constexpr int D = 128;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint4 u = make_uint4(0, 0, 0, 0);
        int d0;
        if (BITS == 4) d0 = 32 * t + 8 * c;
        else d0 = (c < 2 ? 16 * t + 8 * c : 64 + 16 * t + 8 * (c - 2));
        if (g < group) u = *reinterpret_cast<const uint4*>(qrows + (size_t)g * D + d0);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};   // halves d0..d0+7
        if (BITS == 4) {
            // mma 2c: pairs (0,4) (1,5); mma 2c+1: pairs (2,6) (3,7)
            a.qb[2 * c][0] = prmt(w[0], w[2], 0x5410);     a.qb[2 * c][1] = prmt(w[0], w[2], 0x7632);
            a.qb[2 * c + 1][0] = prmt(w[1], w[3], 0x5410); a.qb[2 * c + 1][1] = prmt(w[1], w[3], 0x7632);
        } else {
            // mma 2c: codes 0..3 -> pairs (0,1) (2,3); mma 2c+1: codes 4..7
            a.qb[2 * c][0] = w[0];     a.qb[2 * c][1] = w[1];
            a.qb[2 * c + 1][0] = w[2]; a.qb[2 * c + 1][1] = w[3];
        }
    }
}
// Per-lane source offsets inside a page for kv head h.
struct PageLanes {
    uint32_t k_src0, k_src1, v_src[4], sc_src, sc_dst;
    const __half* sc_base;      // lanes 0-15 copy K scales, lanes 16-31 V scales
};
template <int BITS>
__device__ __forceinline__ PageLanes page_lanes(int lane, int h, uint32_t row_bytes, int scale_row_halves, int Gd,
                                                const __half* k_scales, const __half* v_scales) {
    constexpr int DP = BITS == 4 ? 64 : 128;
    constexpr int K_BYTES = BITS == 4 ? 1024 : 2048;
    const int g = lane >> 2, t = lane & 3;
    PageLanes L;
    L.k_src0 = (uint32_t)g * row_bytes + h * DP + 16 * t;            // token g
    L.k_src1 = L.k_src0 + 8 * row_bytes;                             // token g + 8
#pragma unroll
    for (int i = 0; i < 4; ++i)
        L.v_src[i] = (uint32_t)(2 * t + (i & 1) + 8 * (i >> 1)) * row_bytes + h * DP + (BITS == 4 ? 8 : 16) * g;
    L.sc_src = (uint32_t)(lane & 15) * scale_row_halves + h * Gd;    // halves
    L.sc_dst = 2 * K_BYTES + (lane < 16 ? 0 : 128) + (lane & 15) * 8;
    L.sc_base = lane < 16 ? k_scales : v_scales;
    return L;
}
// Asynchronous copies of one page of kv head h into a ring slot (one commit group, also for a missing page).
template <int BITS, int LOGG>
__device__ __forceinline__ void issue_page(uint8_t* slot, const PageLanes& L, int lane, int page, int valid, const uint8_t* k_codes,
                                           const uint8_t* v_codes, size_t page_code_bytes, size_t page_scale_halves) {
    constexpr int K_BYTES = BITS == 4 ? 1024 : 2048;
    const int g = lane >> 2, t = lane & 3;
    if (page >= 0) {
        const uint8_t* kbase = k_codes + (size_t)page * page_code_bytes;
        const uint8_t* vbase = v_codes + (size_t)page * page_code_bytes;
        if (BITS == 4) {
            // K: 16 bytes of token g and of token g + 8 ; V: 8 bytes of tokens 2t, 2t+1, 2t+8, 2t+9
            if (g < valid) cp_async_16(slot + lane * 16, kbase + L.k_src0);
            if (g + 8 < valid) cp_async_16(slot + 512 + lane * 16, kbase + L.k_src1);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tok = 2 * t + (i & 1) + 8 * (i >> 1);
                if (tok < valid) cp_async_8(slot + K_BYTES + i * 256 + lane * 8, vbase + L.v_src[i]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tok = g + 8 * (i >> 1);
                if (tok < valid)
                    cp_async_16(slot + i * 512 + lane * 16, kbase + (i >> 1 ? L.k_src1 : L.k_src0) + 64 * (i & 1));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tok = 2 * t + (i & 1) + 8 * (i >> 1);
                if (tok < valid) cp_async_16(slot + K_BYTES + i * 512 + lane * 16, vbase + L.v_src[i]);
            }
        }
        // scales of the 16 tokens for this head: lanes 0-15 K, lanes 16-31 V
        if ((lane & 15) < valid) {
            const __half* src = L.sc_base + (size_t)page * page_scale_halves + L.sc_src;
            if (LOGG == 5) cp_async_8(slot + L.sc_dst, src);
            else cp_async_4(slot + L.sc_dst, src);
        }
    }
    cp_async_commit();
}

// One page of kv head h against the group's query heads: S = K Q^T on the tensor cores with the page's 16 tokens as
// rows, online softmax in fp32, O^T += V^T P.  `valid` = tokens of the page below the length (what was copied),
// `attended` = bit mask of the slots that take part.
template <int BITS, int LOGG>
__device__ __forceinline__ void process_page(WarpAcc& a, const uint8_t* slot, int valid, uint32_t attended, float sm_scale,
                                             int lane) {
    constexpr int K_BYTES = BITS == 4 ? 1024 : 2048;
    constexpr int V_BYTES = K_BYTES;
    const int g = lane >> 2;
    const int t = lane & 3;
                const __half* ksc = reinterpret_cast<const __half*>(slot + K_BYTES + V_BYTES);         // [16][4]
        const __half* vsc = ksc + 64;                                                             // [16][4]

        // ---------------- S = K Q^T : rows = tokens g and g + 8, columns = query heads 2t, 2t+1 ----------
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (BITS == 4) {
            const uint4 ua = *reinterpret_cast<const uint4*>(slot + lane * 16);          // token g
            const uint4 ub = *reinterpret_cast<const uint4*>(slot + 512 + lane * 16);    // token g + 8
            const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w}, wb[4] = {ub.x, ub.y, ub.z, ub.w};
            const uint32_t sa = half_dup(__habs(ksc[g * 4 + ((32 * t) >> LOGG)]));
            const uint32_t sb = half_dup(__habs(ksc[(g + 8) * 4 + ((32 * t) >> LOGG)]));
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t wa2 = wa[c] >> 8, wb2 = wb[c] >> 8;
                // exact (code - 8), then one rounding in the multiply: fp16((code-8)*s)
                const uint32_t a0 = hmul2_u32(hsub2_u32(lop3_and_or(wa[c], 0x000F000Fu, 0x64006400u), 0x64086408u), sa);
                const uint32_t a1 = hmul2_u32(hsub2_u32(lop3_and_or(wb[c], 0x000F000Fu, 0x64006400u), 0x64086408u), sb);
                const uint32_t a2 = hmul2_u32(hsub2_u32(lop3_and_or(wa[c], 0x00F000F0u, 0x54005400u), 0x54805480u), sa);
                const uint32_t a3 = hmul2_u32(hsub2_u32(lop3_and_or(wb[c], 0x00F000F0u, 0x54005400u), 0x54805480u), sb);
                mma_m16n8k16(s, a0, a1, a2, a3, a.qb[2 * c][0], a.qb[2 * c][1]);
                const uint32_t c0 = hmul2_u32(hsub2_u32(lop3_and_or(wa2, 0x000F000Fu, 0x64006400u), 0x64086408u), sa);
                const uint32_t c1 = hmul2_u32(hsub2_u32(lop3_and_or(wb2, 0x000F000Fu, 0x64006400u), 0x64086408u), sb);
                const uint32_t c2 = hmul2_u32(hsub2_u32(lop3_and_or(wa2, 0x00F000F0u, 0x54005400u), 0x54805480u), sa);
                const uint32_t c3 = hmul2_u32(hsub2_u32(lop3_and_or(wb2, 0x00F000F0u, 0x54005400u), 0x54805480u), sb);
                mma_m16n8k16(s, c0, c1, c2, c3, a.qb[2 * c + 1][0], a.qb[2 * c + 1][1]);
            }
        } else {
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
                const uint4 ua = *reinterpret_cast<const uint4*>(slot + hb * 512 + lane * 16);          // token g
                const uint4 ub = *reinterpret_cast<const uint4*>(slot + (2 + hb) * 512 + lane * 16);    // token g + 8
                const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w}, wb[4] = {ub.x, ub.y, ub.z, ub.w};
                const uint32_t sa = half_dup(__habs(ksc[g * 4 + ((64 * hb + 16 * t) >> LOGG)]));
                const uint32_t sb = half_dup(__habs(ksc[(g + 8) * 4 + ((64 * hb + 16 * t) >> LOGG)]));
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t a0 = hmul2_u32(hsub2_u32(prmt(wa[c], 0x64646464u, 0x4140u), 0x64806480u), sa);
                    const uint32_t a1 = hmul2_u32(hsub2_u32(prmt(wb[c], 0x64646464u, 0x4140u), 0x64806480u), sb);
                    const uint32_t a2 = hmul2_u32(hsub2_u32(prmt(wa[c], 0x64646464u, 0x4342u), 0x64806480u), sa);
                    const uint32_t a3 = hmul2_u32(hsub2_u32(prmt(wb[c], 0x64646464u, 0x4342u), 0x64806480u), sb);
                    const int mi = 4 * hb + c;
                    mma_m16n8k16(s, a0, a1, a2, a3, a.qb[mi][0], a.qb[mi][1]);
                }
            }
        }
        // ---------------- online softmax: this lane holds heads 2t, 2t+1 of tokens g and g + 8 ----------
        float alpha[2];
        uint32_t pb0, pb1;      // P[token][head] as the B operand of O^T += V^T P
        {
            // also discards whatever stale bytes sit in unused slots
            const bool in0 = (attended >> g) & 1u, in1 = (attended >> (g + 8)) & 1u;
            s[0] = in0 ? s[0] * sm_scale : -INFINITY;
            s[1] = in0 ? s[1] * sm_scale : -INFINITY;
            s[2] = in1 ? s[2] * sm_scale : -INFINITY;
            s[3] = in1 ? s[3] * sm_scale : -INFINITY;
            float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
            for (int o2 = 4; o2 < 32; o2 <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o2));
            }
            const float mn0 = fmaxf(a.m_run[0], mx0), mn1 = fmaxf(a.m_run[1], mx1);   // finite: every staged page has a valid token
            alpha[0] = fast_exp2((a.m_run[0] - mn0) * kLog2e);                       // exp(-inf) = 0 on the first page
            alpha[1] = fast_exp2((a.m_run[1] - mn1) * kLog2e);
            const float p0 = fast_exp2((s[0] - mn0) * kLog2e), p1 = fast_exp2((s[1] - mn1) * kLog2e);
            const float p2 = fast_exp2((s[2] - mn0) * kLog2e), p3 = fast_exp2((s[3] - mn1) * kLog2e);
            // per-lane share of the sums (tokens g, g + 8); the 8 shares of a head are added when a partial is written
            a.l_run[0] = a.l_run[0] * alpha[0] + (p0 + p2);
            a.l_run[1] = a.l_run[1] * alpha[1] + (p1 + p3);
            a.m_run[0] = mn0;
            a.m_run[1] = mn1;
            // transpose (token g, heads 2t, 2t+1) into (tokens 2t, 2t+1, head g): b0b1 tokens 0..7, b2b3 tokens 8..15
            const __half2 x0 = __floats2half2_rn(p0, p1);
            const __half2 x1 = __floats2half2_rn(p2, p3);
            pb0 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&x0));
            pb1 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&x1));
        }
        // ---------------- rescale O^T columns (heads 2t, 2t+1) ----------------------------------------------
        if (__any_sync(0xffffffffu, (alpha[0] != 1.0f) || (alpha[1] != 1.0f))) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                a.o[i][0] *= alpha[0]; a.o[i][1] *= alpha[1]; a.o[i][2] *= alpha[0]; a.o[i][3] *= alpha[1];
            }
        }
        // ---------------- O^T += V^T P ---------------------------------------------------------
        const int vgrp = (16 * g) >> LOGG;
        uint32_t vreg[2][16];   // [token pair][j]: (Vhat[tokA][16g + j], Vhat[tokB][16g + j])
#pragma unroll
        for (int tp = 0; tp < 2; ++tp) {
            const int tokA = 2 * t + 8 * tp, tokB = tokA + 1;
            // slots past the end of the sequence may hold anything: their weight is 0, make the value 0 too
            const __half sA = tokA < valid ? __habs(vsc[tokA * 4 + vgrp]) : __ushort_as_half(0);
            const __half sB = tokB < valid ? __habs(vsc[tokB * 4 + vgrp]) : __ushort_as_half(0);
            const uint32_t s2 = (uint32_t)__half_as_ushort(sA) | ((uint32_t)__half_as_ushort(sB) << 16);
            if (BITS == 4) {
                const uint2 ua = *reinterpret_cast<const uint2*>(slot + K_BYTES + (2 * tp) * 256 + lane * 8);
                const uint2 ub = *reinterpret_cast<const uint2*>(slot + K_BYTES + (2 * tp + 1) * 256 + lane * 8);
                const uint32_t wa[2] = {ua.x, ua.y}, wb[2] = {ub.x, ub.y};
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const uint32_t r0 = prmt(wa[w], wb[w], 0x5410);   // nibbles 0..3 of A | of B
                    const uint32_t r1 = prmt(wa[w], wb[w], 0x7632);   // nibbles 4..7
                    const uint32_t r0s = r0 >> 8, r1s = r1 >> 8;
                    vreg[tp][8 * w + 0] = hmul2_u32(hsub2_u32(lop3_and_or(r0, 0x000F000Fu, 0x64006400u), 0x64086408u), s2);
                    vreg[tp][8 * w + 1] = hmul2_u32(hsub2_u32(lop3_and_or(r0, 0x00F000F0u, 0x54005400u), 0x54805480u), s2);
                    vreg[tp][8 * w + 2] = hmul2_u32(hsub2_u32(lop3_and_or(r0s, 0x000F000Fu, 0x64006400u), 0x64086408u), s2);
                    vreg[tp][8 * w + 3] = hmul2_u32(hsub2_u32(lop3_and_or(r0s, 0x00F000F0u, 0x54005400u), 0x54805480u), s2);
                    vreg[tp][8 * w + 4] = hmul2_u32(hsub2_u32(lop3_and_or(r1, 0x000F000Fu, 0x64006400u), 0x64086408u), s2);
                    vreg[tp][8 * w + 5] = hmul2_u32(hsub2_u32(lop3_and_or(r1, 0x00F000F0u, 0x54005400u), 0x54805480u), s2);
                    vreg[tp][8 * w + 6] = hmul2_u32(hsub2_u32(lop3_and_or(r1s, 0x000F000Fu, 0x64006400u), 0x64086408u), s2);
                    vreg[tp][8 * w + 7] = hmul2_u32(hsub2_u32(lop3_and_or(r1s, 0x00F000F0u, 0x54005400u), 0x54805480u), s2);
                }
            } else {
                const uint4 ua = *reinterpret_cast<const uint4*>(slot + K_BYTES + (2 * tp) * 512 + lane * 16);
                const uint4 ub = *reinterpret_cast<const uint4*>(slot + K_BYTES + (2 * tp + 1) * 512 + lane * 16);
                const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w}, wb[4] = {ub.x, ub.y, ub.z, ub.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t e = prmt(wa[w], wb[w], 0x5140);   // A.b0 B.b0 A.b1 B.b1
                    const uint32_t f2 = prmt(wa[w], wb[w], 0x7362);  // A.b2 B.b2 A.b3 B.b3
                    vreg[tp][4 * w + 0] = hmul2_u32(hsub2_u32(prmt(e, 0x64646464u, 0x4140u), 0x64806480u), s2);
                    vreg[tp][4 * w + 1] = hmul2_u32(hsub2_u32(prmt(e, 0x64646464u, 0x4342u), 0x64806480u), s2);
                    vreg[tp][4 * w + 2] = hmul2_u32(hsub2_u32(prmt(f2, 0x64646464u, 0x4140u), 0x64806480u), s2);
                    vreg[tp][4 * w + 3] = hmul2_u32(hsub2_u32(prmt(f2, 0x64646464u, 0x4342u), 0x64806480u), s2);
                }
            }
        }
        // tile i: row g <-> d = 16g + 2i, row g+8 <-> d = 16g + 2i + 1
#pragma unroll
        for (int i = 0; i < 8; ++i)
            mma_m16n8k16(a.o[i], vreg[0][2 * i], vreg[0][2 * i + 1], vreg[1][2 * i], vreg[1][2 * i + 1], pb0, pb1);
}

// Two shapes of the same kernel.  TWO = true: two CTAs per SM (16 warps hide more of the dequantisation
// latency: 41 us against 45 us on the batch-16 q4 case) with the ring depth that still fits twice into shared
// memory.  TWO = false: one CTA per SM with a deeper ring, for grids that do not fill the SMs twice anyway.
constexpr int ring_depth(int bits, bool two) { return bits == 4 ? (two ? 4 : 8) : (two ? 2 : 5); }
template <int BITS, int LOGG, bool TWO>
__global__ void __launch_bounds__(kAttnThreads, TWO ? B200Q_ATTN_CTAS : 1) paged_attn_kernel(const __grid_constant__ AttnParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int D = 128;
    constexpr int K_BYTES = BITS == 4 ? 1024 : 2048;  // per page and head
    constexpr int V_BYTES = K_BYTES;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    int* prefix = reinterpret_cast<int*>(smem + p.off_prefix);   // [B + 1]

    pdl_launch_dependents();
    pdl_wait();   // lengths / block table / q / the cache itself may be produced by the previous kernel

    // The flattened page list is cut into p.grid equal ranges.  A CTA has 8 warps = 8 (range, kv head) pairs:
    // with 8 kv heads one range, with fewer heads several consecutive ranges (subs of them).  The cut depends
    // only on the batch and the device, not on the number of heads, so a head's partial results (and the
    // merged output) are the same bits whether all heads or a tensor-parallel shard of them are computed.
    const int total = build_prefix(p, prefix);
    const int ppc = (total + p.grid - 1) / p.grid;               // pages per range
    const int subs = p.subs;
    const int h = warp % p.Hkv;                                  // kv head of this warp
    const int sub = warp / p.Hkv;
    const int vc = (int)blockIdx.x * subs + sub;                 // range of this warp
    const int lo = min(total, vc * ppc);
    const int hi = min(total, lo + ppc);
    if (lo >= hi || sub >= subs || vc >= p.grid) return;

    const int g = lane >> 2;
    const int t = lane & 3;
    const int group = p.group;
    const float sm_scale = p.scale;
    constexpr int NS = ring_depth(BITS, TWO);                     // pages in flight per warp
    constexpr int SLOT = K_BYTES + V_BYTES + 256;                // bytes of one ring slot
    uint8_t* my_ring = smem + p.off_ring + (size_t)warp * NS * SLOT;
    const int n_my = hi - lo;                                     // pages this warp walks: f = lo + j

    WarpAcc acc;
    acc_reset(acc);
    int cur_b = -1;

    // Page descriptors (page id, sequence, valid tokens) of 32 consecutive pages of this warp, one per
    // lane.  Two windows: one for the page being consumed, one for the page being issued ahead.
    struct Desc { int page, b, valid; };      // valid: token count | attended-slot mask << 16
    auto lookup = [&](int base) -> Desc {
        const int j = base + lane;
        Desc d = {-1, 0, 0};
        if (j < n_my) {
            const int f = lo + j;
            const int b = find_sequence(prefix, p.B, f);
            const SeqPages sp = seq_pages(p.lengths[b], p.max_blocks * p.P, p.P, p.sink, p.window);
            const int idx = f - prefix[b];
            const int pg = idx < sp.sink_pages ? idx : sp.first_recent + (idx - sp.sink_pages);
            int page = p.block_table[(int64_t)b * p.max_blocks + pg];
            if (page < 0 || page >= p.num_pages) page = -1;
            d.page = page;
            d.b = b;
            // low half: tokens of the page below the length (what is copied); high half: attended slots
            d.valid = min(p.P, sp.L - pg * p.P) | (int)(page_mask16(pg, sp.L, p.sink, p.window) << 16);
        }
        return d;
    };
    Desc win_c = lookup(0);     // consume window
    Desc win_i = win_c;         // issue window
    const PageLanes L = page_lanes<BITS>(lane, h, (uint32_t)p.row_bytes, p.scale_row_halves, p.Gd, p.k_scales, p.v_scales);
    const size_t page_code_bytes = (size_t)p.P * p.row_bytes;
    const size_t page_scale_halves = (size_t)p.P * p.scale_row_halves;
    int slot_i = 0;      // ring slot of the next page to issue
    // issue the asynchronous copies of page j (descriptor held by lane j % 32 of the issue window)
    auto issue = [&](int j) {
        if (j > 0 && (j & 31) == 0) win_i = lookup(j);
        const int src_lane = j & 31;
        const int page = __shfl_sync(0xffffffffu, win_i.page, src_lane);
        const int valid = __shfl_sync(0xffffffffu, win_i.valid, src_lane) & 0xFFFF;
        issue_page<BITS, LOGG>(my_ring + slot_i * SLOT, L, lane, page, valid, p.k_codes, p.v_codes, page_code_bytes,
                               page_scale_halves);
        slot_i = (slot_i + 1 == NS) ? 0 : slot_i + 1;
    };

    auto flush = [&](int b) {
        float* dst = p.partial + ((size_t)(vc + b) * p.Hq) * (D + 2);
        float l0 = acc.l_run[0], l1 = acc.l_run[1];
#pragma unroll
        for (int o2 = 4; o2 < 32; o2 <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, o2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, o2);
        }
        // O^T[d][head]: thread (g,t) holds d = 16g + 2i (+1), heads 2t, 2t+1
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int head = 2 * t + (e & 1);
                const int d = 16 * g + 2 * i + (e >> 1);
                if (head < group) dst[(size_t)(h * group + head) * (D + 2) + d] = acc.o[i][e];
            }
        }
        if (g == 0) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int head = 2 * t + e;
                if (head < group) {
                    dst[(size_t)(h * group + head) * (D + 2) + D] = acc.m_run[e];
                    dst[(size_t)(h * group + head) * (D + 2) + D + 1] = e ? l1 : l0;
                }
            }
        }
    };

    // prologue: copies of the first NS - 1 pages
    for (int j = 0; j < NS - 1; ++j) {
        if (j < n_my) issue(j);
        else { cp_async_commit(); slot_i = (slot_i + 1 == NS) ? 0 : slot_i + 1; }
    }

    int slot_c = 0;     // ring slot of the page being consumed
    for (int j = 0; j < n_my; ++j) {
        if (j > 0 && (j & 31) == 0) win_c = lookup(j);
        const int page = __shfl_sync(0xffffffffu, win_c.page, j & 31);
        const int b = __shfl_sync(0xffffffffu, win_c.b, j & 31);
        const uint32_t valid_mask = (uint32_t)__shfl_sync(0xffffffffu, win_c.valid, j & 31);
        const int valid = (int)(valid_mask & 0xFFFFu);
        const uint32_t attended = valid_mask >> 16;
        // look-ahead: copies of page j + NS - 1 (an empty group keeps the count uniform at the end)
        if (j + NS - 1 < n_my) issue(j + NS - 1);
        else cp_async_commit();
        cp_async_wait<NS - 1>();     // at most NS - 1 groups pending: page j has landed
        __syncwarp();

        if (b != cur_b) {
            if (cur_b >= 0) flush(cur_b);
            cur_b = b;
            acc_reset(acc);
            load_q_frags<BITS>(acc, p.q + ((size_t)b * p.Hq + h * group) * D, group, g, t);
        }
        if (page >= 0) process_page<BITS, LOGG>(acc, my_ring + slot_c * SLOT, valid, attended, sm_scale, lane);
        __syncwarp();   // every lane is done with this slot before it is refilled
        slot_c = (slot_c + 1 == NS) ? 0 : slot_c + 1;
    }
    if (cur_b >= 0) flush(cur_b);
}

// ------------------------------------------------------------------------------------------------
// Cluster kernel for small batches: one thread-block cluster per (sequence, kv head), no partials in global memory
// and no merge launch.  The CTAs of the cluster cut the sequence's pages into equal ranges, the 8 warps of a CTA cut
// their range again; a warp walks its pages exactly as in the split-KV kernel.  The warps' partial (max, sum,
// accumulator) triples are merged in shared memory, the CTAs' through distributed shared memory by the cluster's
// first CTA, always in the same order (bitwise repeatable, and independent of how many kv heads a tensor-parallel
// shard holds).  Optionally the kernel also does what precedes attention in a decode layer - split the fused QKV
// row, rotate q and k, quantise and append the new token's k / v to its page: the CTA that walks the page of the
// new position appends kv head h itself before it reads that page, every CTA rotates its own copy of q.
// ------------------------------------------------------------------------------------------------
struct ClusterAttnParams {
    const __half* q;            // [B, Hq, D] rotated queries (fused == 0)
    const __half* qkv;          // fused: [B, (Hq + 2 Hkv) * D]
    const float* cos_table;     // fused: [table_len, D/2]
    const float* sin_table;
    const int32_t* positions;   // fused: [B]
    uint8_t* k_codes;
    uint8_t* v_codes;
    __half* k_scales;
    __half* v_scales;
    const int32_t* block_table;
    const int32_t* lengths;
    void* out;                  // [B, Hq, D]
    int B, Hq, Hkv, P, max_blocks, G, Gd, group, bits, table_len, fused, S;
    int64_t num_pages;
    float scale;
    int row_bytes, scale_row_halves;
    uint32_t off_q, off_wpart, off_cpart, off_ring;
    TpOut tp_out;
};

__device__ __forceinline__ uint32_t cluster_rank_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

template <int BITS, int LOGG>
__global__ void __launch_bounds__(kAttnThreads, 1) paged_attn_cluster_kernel(const __grid_constant__ ClusterAttnParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int D = 128;
    constexpr int K_BYTES = BITS == 4 ? 1024 : 2048;
    constexpr int V_BYTES = K_BYTES;
    constexpr int NS = BITS == 4 ? 8 : 5;                         // pages in flight per warp
    constexpr int SLOT = K_BYTES + V_BYTES + 256;
    constexpr int PW = D + 2;                                     // floats of one partial: accumulator, max, sum
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t rank = cluster_rank_x();
    const int h = blockIdx.y;
    const int b = blockIdx.z;
    const int group = p.group;
    const int S = p.S;
    __half* qs = reinterpret_cast<__half*>(smem + p.off_q);              // [group][D] rotated query rows
    float* wpart = reinterpret_cast<float*>(smem + p.off_wpart);         // [8 warps][group][PW]
    float* cpart = reinterpret_cast<float*>(smem + p.off_cpart);         // [S][group][PW] (used in the first CTA)

    pdl_launch_dependents();
    pdl_wait();

    const int L = clamp_len(p.lengths[b], p.max_blocks * p.P);
    const int n_pages = (L + p.P - 1) / p.P;
    const int ppc = (n_pages + S - 1) / S;                               // pages per CTA
    const int c_lo = min(n_pages, (int)rank * ppc), c_hi = min(n_pages, c_lo + ppc);
    const int ppw = (c_hi - c_lo + kAttnWarps - 1) / kAttnWarps;         // pages per warp
    const int lo = min(c_hi, c_lo + warp * ppw), hi = min(c_hi, lo + ppw);

    if (p.fused) {
        const int heads = p.Hq + 2 * p.Hkv;
        const int pos = p.positions[b];
        const bool pos_ok = pos >= 0 && pos < p.table_len;
        const int d0 = lane * 4;
        const __half* row = p.qkv + (size_t)b * heads * D;
        auto load4 = [&](int head, float (&v)[4]) {
            const uint2 u = *reinterpret_cast<const uint2*>(row + (size_t)head * D + d0);
            const __half2 h0 = *reinterpret_cast<const __half2*>(&u.x), h1 = *reinterpret_cast<const __half2*>(&u.y);
            v[0] = __low2float(h0); v[1] = __high2float(h0); v[2] = __low2float(h1); v[3] = __high2float(h1);
        };
        auto rope4 = [&](float (&v)[4]) {
            if (!pos_ok) return;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float c = p.cos_table[(size_t)pos * (D / 2) + d0 / 2 + i];
                const float sn = p.sin_table[(size_t)pos * (D / 2) + d0 / 2 + i];
                const float xe = v[2 * i], xo = v[2 * i + 1];
                // two separately rounded products and one sum, as the reference's elementwise expression
                v[2 * i] = __fsub_rn(__fmul_rn(xe, c), __fmul_rn(xo, sn));
                v[2 * i + 1] = __fadd_rn(__fmul_rn(xe, sn), __fmul_rn(xo, c));
            }
        };
        if (!pos_ok && threadIdx.x == 0) atomicMax(&g_device_status, (int)EV_ROPE_POSITION);
        // rotated query rows of this kv head's group, one warp per query head
        if (warp < group) {
            float v[4];
            load4(h * group + warp, v);
            rope4(v);
            const __half2 a0 = __floats2half2_rn(v[0], v[1]), a1 = __floats2half2_rn(v[2], v[3]);
            uint2 o2;
            o2.x = *reinterpret_cast<const uint32_t*>(&a0);
            o2.y = *reinterpret_cast<const uint32_t*>(&a1);
            *reinterpret_cast<uint2*>(qs + (size_t)warp * D + d0) = o2;
        }
        // append k (rotated) and v of kv head h to the page of `pos`: the CTA whose range holds that page
        const int blk = pos >= 0 ? pos / p.P : -1;
        const int owner = (ppc > 0 && blk >= 0) ? min(S - 1, blk / ppc) : 0;
        if ((int)rank == owner && warp >= 6) {
            const bool is_v = warp == 7;
            int page = (blk >= 0 && blk < p.max_blocks) ? p.block_table[(size_t)b * p.max_blocks + blk] : -1;
            if (page < 0 || page >= p.num_pages) {
                if (lane == 0) atomicMax(&g_device_status, (int)EV_KV_PAGE_UNASSIGNED);
            } else {
                float v[4];
                load4(p.Hq + (is_v ? p.Hkv : 0) + h, v);
                if (!is_v) rope4(v);
                __half hv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) { hv[i] = __float2half_rn(v[i]); v[i] = __half2float(hv[i]); }
                float mx = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
                const int lanes_per_group = p.G / 4;
                for (int o2 = 1; o2 < lanes_per_group; o2 <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
                const float limit = BITS == 8 ? 127.0f : 7.0f;
                const float offset = BITS == 8 ? 128.0f : 8.0f;
                const float sc = __fdiv_rn(fmaxf(mx, 1e-8f), limit);
                uint32_t codes[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    codes[i] = (uint32_t)(int)(fminf(fmaxf(rintf(__fdiv_rn(v[i], sc)), -limit), limit) + offset);
                const size_t tok = ((size_t)page * p.P + (pos % p.P)) * p.Hkv + h;
                uint8_t* cdst = is_v ? p.v_codes : p.k_codes;
                __half* sdst = is_v ? p.v_scales : p.k_scales;
                if (BITS == 8)
                    *reinterpret_cast<uint32_t*>(cdst + tok * D + d0) = codes[0] | (codes[1] << 8) | (codes[2] << 16) | (codes[3] << 24);
                else
                    *reinterpret_cast<uint16_t*>(cdst + tok * (D / 2) + d0 / 2) =
                        (uint16_t)(codes[0] | (codes[1] << 4) | (codes[2] << 8) | (codes[3] << 12));
                if ((lane % lanes_per_group) == 0) sdst[tok * p.Gd + d0 / p.G] = __float2half_rn(sc);
            }
            __threadfence();          // the appended bytes are in global memory before this CTA's copies read the page
        }
        __syncthreads();
    }

    // ---- this warp's pages ----
    WarpAcc acc;
    acc_reset(acc);
    const int n_my = hi - lo;
    if (n_my > 0) {
        const __half* qrows = p.fused ? qs : p.q + ((size_t)b * p.Hq + h * group) * D;
        load_q_frags<BITS>(acc, qrows, group, g, t);
        const PageLanes Lp = page_lanes<BITS>(lane, h, (uint32_t)p.row_bytes, p.scale_row_halves, p.Gd, p.k_scales, p.v_scales);
        const size_t page_code_bytes = (size_t)p.P * p.row_bytes;
        const size_t page_scale_halves = (size_t)p.P * p.scale_row_halves;
        uint8_t* my_ring = smem + p.off_ring + (size_t)warp * NS * SLOT;
        auto page_of = [&](int j) -> int {
            int page = p.block_table[(size_t)b * p.max_blocks + lo + j];
            return (page < 0 || page >= p.num_pages) ? -1 : page;
        };
        auto valid_of = [&](int j) -> int { return min(p.P, L - (lo + j) * p.P); };
        int slot_i = 0, slot_c = 0;
        for (int j = 0; j < NS - 1; ++j) {
            if (j < n_my) issue_page<BITS, LOGG>(my_ring + slot_i * SLOT, Lp, lane, page_of(j), valid_of(j), p.k_codes, p.v_codes,
                                                 page_code_bytes, page_scale_halves);
            else cp_async_commit();
            slot_i = (slot_i + 1 == NS) ? 0 : slot_i + 1;
        }
        for (int j = 0; j < n_my; ++j) {
            if (j + NS - 1 < n_my)
                issue_page<BITS, LOGG>(my_ring + slot_i * SLOT, Lp, lane, page_of(j + NS - 1), valid_of(j + NS - 1), p.k_codes,
                                       p.v_codes, page_code_bytes, page_scale_halves);
            else cp_async_commit();
            slot_i = (slot_i + 1 == NS) ? 0 : slot_i + 1;
            cp_async_wait<NS - 1>();
            __syncwarp();
            const int valid = valid_of(j);
            const uint32_t attended = valid >= 16 ? 0xFFFFu : ((1u << max(valid, 0)) - 1u);
            if (page_of(j) >= 0) process_page<BITS, LOGG>(acc, my_ring + slot_c * SLOT, valid, attended, p.scale, lane);
            __syncwarp();
            slot_c = (slot_c + 1 == NS) ? 0 : slot_c + 1;
        }
    }
    // ---- the warp's partial: O^T[d][head] with thread (g,t) holding d = 16g + 2i (+1), heads 2t, 2t+1 ----
    {
        float l0 = acc.l_run[0], l1 = acc.l_run[1];
#pragma unroll
        for (int o2 = 4; o2 < 32; o2 <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, o2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, o2);
        }
        float* dst = wpart + (size_t)warp * group * PW;
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int head = 2 * t + (e & 1);
                if (head < group) dst[head * PW + 16 * g + 2 * i + (e >> 1)] = acc.o[i][e];
            }
        if (g == 0) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int head = 2 * t + e;
                if (head < group) {
                    dst[head * PW + D] = acc.m_run[e];
                    dst[head * PW + D + 1] = e ? l1 : l0;
                }
            }
        }
    }
    __syncthreads();
    // ---- merge the 8 warps (fixed order) into this CTA's partial; thread -> (head, d) ----
    auto merge = [&](const float* src, int n, int head, int d, float& m_tot, float& l_tot) -> float {
        m_tot = -INFINITY;
        for (int i = 0; i < n; ++i) m_tot = fmaxf(m_tot, src[((size_t)i * group + head) * PW + D]);
        float accv = 0.0f;
        l_tot = 0.0f;
        for (int i = 0; i < n; ++i) {
            const float* ps = src + ((size_t)i * group + head) * PW;
            const float m = ps[D];
            const float w = m == -INFINITY ? 0.0f : exp2f((m - m_tot) * kLog2e);
            accv = fmaf(w, ps[d], accv);
            l_tot = fmaf(w, ps[D + 1], l_tot);
        }
        return accv;
    };
    const uint32_t cpart_u = smem_u32(cpart);
    for (int idx = threadIdx.x; idx < group * D; idx += kAttnThreads) {
        const int head = idx / D, d = idx - head * D;
        float m_tot, l_tot;
        const float v = merge(wpart, kAttnWarps, head, d, m_tot, l_tot);
        // slot `rank` of the first CTA's table (its own slot for the first CTA itself)
        const uint32_t base = cpart_u + (uint32_t)((rank * group + head) * PW) * 4u;
        auto put = [&](uint32_t off, float val) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(base + off * 4u), "r"(0));
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(val) : "memory");
        };
        put((uint32_t)d, v);
        if (d == 0) { put((uint32_t)D, m_tot); put((uint32_t)D + 1, l_tot); }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank == 0) {
        for (int idx = threadIdx.x; idx < group * D; idx += kAttnThreads) {
            const int head = idx / D, d = idx - head * D;
            float m_tot, l_tot;
            const float v = merge(cpart, S, head, d, m_tot, l_tot);
            const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
            const unsigned short bits16 = __half_as_ushort(__float2half_rn(v * inv));
            const int hq = h * group + head;
            if (p.out != nullptr) reinterpret_cast<unsigned short*>(p.out)[((size_t)b * p.Hq + hq) * D + d] = bits16;
            if (p.tp_out.world > 0) {
                const size_t of = ((size_t)b * p.tp_out.world + p.tp_out.rank) * p.Hq * D + (size_t)hq * D + d;
                if (p.tp_out.packets) {
                    const uint32_t pk = tp_packet(bits16, tp_seq16(tp_writer_seq(p.tp_out)));
#pragma unroll 1
                    for (int peer = 0; peer < p.tp_out.world; ++peer)
                        st_volatile_u32(reinterpret_cast<uint32_t*>(p.tp_out.full[peer]) + of, pk);
                } else {
#pragma unroll 1
                    for (int peer = 0; peer < p.tp_out.world; ++peer)
                        reinterpret_cast<unsigned short*>(p.tp_out.full[peer])[of] = bits16;
                }
            }
        }
    }
    if (p.tp_out.world > 0) {
        __syncthreads();                         // all of this CTA's peer stores are issued
        if (warp == 0) {
            if (p.tp_out.packets) tp_finish_writer_packets(p.tp_out, lane, gridDim.x * gridDim.y * gridDim.z);
            else tp_finish_writer(p.tp_out, lane, gridDim.x * gridDim.y * gridDim.z);
        }
    }
}

// Merges the partials of every (sequence, query head): one warp each, lanes over d.

// One CTA per (sequence, query head).  The partials of a sequence may sit in every CTA slot of the
// main kernel (a single long sequence is cut over the whole grid), so the slots are spread over the
// CTA's warps and their loads are independent of one another; lanes cover the head dimension.
// kMergeWarps: 32 for short batches (few CTAs, up to ~300 candidates each: four loads in flight per warp cover
// them in one or two rounds), 8 for long batches (many CTAs with a dozen candidates each).
template <int kMergeWarps>
__global__ void __launch_bounds__(kMergeWarps * 32) paged_attn_merge_kernel(const __grid_constant__ AttnParams p) {
    __shared__ float red[kMergeWarps][128];
    __shared__ float red_s[2][kMergeWarps];
    __shared__ int red_i[2][kMergeWarps];
    __shared__ int cand_off[kMaxGrid];            // candidates: page ranges of the main kernel that touch this sequence
    __shared__ float cand_m[kMaxGrid];
    const int D = p.D;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int b = blockIdx.x / p.Hq;
    const int hq = blockIdx.x - b * p.Hq;
    pdl_wait();

    // pages before sequence b and in total (the flattened page list of the main kernel)
    const int cap = p.max_blocks * p.P;
    int below = 0, all = 0;
    for (int i = threadIdx.x; i < p.B; i += kMergeWarps * 32) {
        const int n = seq_pages(p.lengths[i], cap, p.P, p.sink, p.window).n;
        all += n;
        if (i < b) below += n;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        below += __shfl_xor_sync(0xffffffffu, below, o);
        all += __shfl_xor_sync(0xffffffffu, all, o);
    }
    if (lane == 0) { red_i[0][warp] = below; red_i[1][warp] = all; }
    __syncthreads();
    below = 0; all = 0;
#pragma unroll
    for (int w = 0; w < kMergeWarps; ++w) { below += red_i[0][w]; all += red_i[1][w]; }
    const int total = all;
    const int s_lo = below;
    const int s_hi = below + seq_pages(p.lengths[b], cap, p.P, p.sink, p.window).n;
    const int ppc = (total + p.grid - 1) / p.grid;

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float l_part = 0.0f;
    if (s_hi > s_lo) {
        const int c_first = s_lo / ppc, c_last = (s_hi - 1) / ppc;
        const int n_cand = c_last - c_first + 1;
        // Every range c_first..c_last holds at least one page of b, i.e. wrote a partial into slot c + b.
        // Pass 1 (one candidate per thread): the offset of the partial and its running maximum, kept in shared
        // memory so that pass 2 is free of index arithmetic.
        float m_tot = -INFINITY;
        for (int i = threadIdx.x; i < n_cand; i += kMergeWarps * 32) {
            const int off = ((c_first + i + b) * p.Hq + hq) * (D + 2);
            const float m = p.partial[(size_t)off + D];
            cand_off[i] = off;
            cand_m[i] = m;
            m_tot = fmaxf(m_tot, m);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m_tot = fmaxf(m_tot, __shfl_xor_sync(0xffffffffu, m_tot, o));
        if (lane == 0) red_s[0][warp] = m_tot;
        __syncthreads();
#pragma unroll
        for (int w = 0; w < kMergeWarps; ++w) m_tot = fmaxf(m_tot, red_s[0][w]);

#pragma unroll 4
        for (int i = warp; i < n_cand; i += kMergeWarps) {
            const int off = cand_off[i];
            const float m = cand_m[i];
            const bool ok = off >= 0 && m != -INFINITY;
            const float* src = p.partial + (ok ? off : 0);
            const float w = ok ? exp2f((m - m_tot) * kLog2e) : 0.0f;
            const float l = ok ? src[D + 1] : 0.0f;
            l_part = fmaf(w, l, l_part);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int d = lane + 32 * j;
                const float v = (ok && d < D) ? src[d] : 0.0f;
                acc[j] = fmaf(w, v, acc[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) red[warp][lane + 32 * j] = acc[j];
    if (lane == 0) red_s[1][warp] = l_part;
    __syncthreads();
    if (threadIdx.x < D) {
        float sum = 0.0f, l_tot = 0.0f;
#pragma unroll
        for (int w = 0; w < kMergeWarps; ++w) { sum += red[w][threadIdx.x]; l_tot += red_s[1][w]; }
        const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
        const size_t o = ((size_t)b * p.Hq + hq) * D + threadIdx.x;
        const unsigned short bits16 = p.q_dtype == B200Q_F16 ? __half_as_ushort(__float2half_rn(sum * inv))
                                                             : __bfloat16_as_ushort(__float2bfloat16_rn(sum * inv));
        if (p.out != nullptr) reinterpret_cast<unsigned short*>(p.out)[o] = bits16;
        if (p.tp_out.world > 0) {
            // tensor-parallel exchange: this head's row goes to column block `rank` of every rank's full rows
            const size_t of = ((size_t)b * p.tp_out.world + p.tp_out.rank) * p.Hq * D + (size_t)hq * D + threadIdx.x;
            if (p.tp_out.packets) {
                const uint32_t pk = tp_packet(bits16, tp_seq16(tp_writer_seq(p.tp_out)));
#pragma unroll 1
                for (int peer = 0; peer < p.tp_out.world; ++peer)
                    st_volatile_u32(reinterpret_cast<uint32_t*>(p.tp_out.full[peer]) + of, pk);
            } else {
#pragma unroll 1
                for (int peer = 0; peer < p.tp_out.world; ++peer)
                    reinterpret_cast<unsigned short*>(p.tp_out.full[peer])[of] = bits16;
            }
        }
    }
    if (p.tp_out.world > 0) {
        __syncthreads();                         // all of this CTA's peer stores are issued
        if (warp == 0) {
            if (p.tp_out.packets) tp_finish_writer_packets(p.tp_out, lane);
            else tp_finish_writer(p.tp_out, lane);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Simple kernel: one warp per (b, hq); any D <= 128, any group size, fp16/bf16 q, any scale dtype.
// ------------------------------------------------------------------------------------------------
struct SimpleParams {
    const void* q; const uint8_t* k_codes; const uint8_t* v_codes; const void* k_scales; const void* v_scales;
    const int32_t* block_table; const int32_t* lengths; void* out;
    int B, Hq, Hkv, D, P, max_blocks, G, Gd, bits, q_dtype, scale_dtype;
    int64_t num_pages;
    float scale;
    int sink, window;
    const uint8_t* block_mask;      // block-sparse decode: [n_qblocks, n_kblocks] bytes, or null
    int block_size, n_qblocks, n_kblocks;
};

__global__ void __launch_bounds__(128) paged_attn_simple_kernel(const __grid_constant__ SimpleParams p) {
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= p.B * p.Hq) return;
    const int b = item / p.Hq;
    const int hq = item - b * p.Hq;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int DPk = p.bits == 4 ? (p.D + 1) / 2 : p.D;
    const int L = clamp_len(p.lengths[b], p.max_blocks * p.P);
    float qv[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int d = lane + 32 * j;
        qv[j] = d < p.D ? load_as_f32(p.q, p.q_dtype, ((int64_t)b * p.Hq + hq) * p.D + d) : 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    const float off = p.bits == 4 ? 8.0f : 128.0f;
    // block-sparse: the query sits at position L - 1, i.e. in row (L - 1) / block_size of the mask
    const int qb = (p.block_mask != nullptr && L > 0) ? (L - 1) / p.block_size : 0;
    const uint8_t* mask_row = (p.block_mask != nullptr && qb < p.n_qblocks) ? p.block_mask + (size_t)qb * p.n_kblocks : nullptr;
    for (int j = 0; j < L; ++j) {
        if (p.window > 0 && j >= p.sink && j < L - p.window) continue;     // outside sink and window
        if (p.block_mask != nullptr) {
            const int kb = j / p.block_size;
            if (mask_row == nullptr || kb >= p.n_kblocks || mask_row[kb] == 0) continue;
        }
        const int page = p.block_table[(int64_t)b * p.max_blocks + j / p.P];
        if (page < 0 || page >= p.num_pages) continue;
        const int64_t tok = ((int64_t)page * p.P + (j % p.P)) * p.Hkv + hkv;
        float kd[4], vd[4], dot = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = lane + 32 * i;
            kd[i] = vd[i] = 0.0f;
            if (d < p.D) {
                uint32_t kc, vc;
                if (p.bits == 4) {
                    const uint8_t kb = p.k_codes[tok * DPk + (d >> 1)], vb = p.v_codes[tok * DPk + (d >> 1)];
                    kc = (d & 1) ? (kb >> 4) : (kb & 0xF);
                    vc = (d & 1) ? (vb >> 4) : (vb & 0xF);
                } else {
                    kc = p.k_codes[tok * DPk + d];
                    vc = p.v_codes[tok * DPk + d];
                }
                const float ks = fabsf(load_as_f32(p.k_scales, p.scale_dtype, tok * p.Gd + d / p.G));
                const float vs = fabsf(load_as_f32(p.v_scales, p.scale_dtype, tok * p.Gd + d / p.G));
                kd[i] = __half2float(__float2half_rn(__fmul_rn((float)kc - off, ks)));
                vd[i] = __half2float(__float2half_rn(__fmul_rn((float)vc - off, vs)));
                dot = fmaf(qv[i], kd[i], dot);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float sc = dot * p.scale;
        const float m_new = fmaxf(m, sc);
        const float alpha = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        const float beta = expf(sc - m_new);
        l = l * alpha + beta;
        m = m_new;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = acc[i] * alpha + beta * vd[i];
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int d = lane + 32 * i;
        if (d < p.D) {
            const int64_t o = ((int64_t)b * p.Hq + hq) * p.D + d;
            if (p.q_dtype == B200Q_F16) reinterpret_cast<__half*>(p.out)[o] = __float2half_rn(acc[i] * inv);
            else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(acc[i] * inv);
        }
    }
}

inline uint32_t align_up_u32(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }
inline int subs_for(int Hkv) { return (Hkv <= kAttnWarps && kAttnWarps % Hkv == 0) ? kAttnWarps / Hkv : 1; }

// ---- cluster kernel: host side ----
int cluster_size_for(int B, int Hkv) {
    const int mode = tuning_get("attn.cluster");      // 1: whenever possible, -1: never, 0: small batches
    if (mode < 0) return 0;
    const int pairs = B * Hkv;
    const int sms = sm_count();
    // the choice follows the kv heads of the UNSHARDED cache ("ts.tp_world" equal head shards), so that a
    // tensor-parallel rank runs the same kernel, and the same summation order, as the unsharded call
    if (mode == 0 && pairs * std::max(1, tuning_get("ts.tp_world")) * 8 > 2 * sms) return 0;
    if (mode > 0 && pairs > 65535) return 0;
    // 8 CTAs per cluster; the opt-in size 16 measured slower (placing one cluster per GPC costs more than the shorter
    // page walk saves: 17.8 us against 12.9 us per stage at batch 1, context 4096)
    int size = 8;
    const int forced = tuning_get("attn.cluster_size");
    if (forced == 8 || forced == 16 || forced == 4) size = forced;
    return size;
}

int launch_cluster_attention(ClusterAttnParams& p, cudaStream_t stream) {
    const bool g32 = p.G == 32;
    const int slot = (p.bits == 4 ? 2048 : 4096) + 256;
    const int ns = p.bits == 4 ? 8 : 5;
    uint32_t off = 0;
    p.off_q = off;      off += align_up_u32((uint32_t)p.group * 128 * 2, 128);
    p.off_wpart = off;  off += align_up_u32((uint32_t)kAttnWarps * p.group * 130 * 4, 128);
    p.off_cpart = off;  off += align_up_u32((uint32_t)p.S * p.group * 130 * 4, 128);
    p.off_ring = off;   off += (uint32_t)kAttnWarps * ns * slot;
    const uint32_t cap = (uint32_t)max_smem_optin();
    if (off > cap) return B200Q_ERR_UNSUPPORTED;
    using KernelFn = void (*)(ClusterAttnParams);
    KernelFn kernel = p.bits == 4 ? (g32 ? paged_attn_cluster_kernel<4, 5> : paged_attn_cluster_kernel<4, 6>)
                                  : (g32 ? paged_attn_cluster_kernel<8, 5> : paged_attn_cluster_kernel<8, 6>);
    static bool configured[2][2][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[p.bits == 4][g32][dev & 63]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap) != cudaSuccess ||
            cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
            return B200Q_ERR_LAUNCH;
        configured[p.bits == 4][g32][dev & 63] = true;
    }
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (!tuning_get("no_pdl")) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = p.S;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.S, p.Hkv, p.B);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = off;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return B200Q_ERR_LAUNCH;
    return finish_launch();
}

}  // namespace

int attention_stage_launches_impl(int B, int Hkv, int with_append) {
    if (B <= 0 || Hkv <= 0) return 0;
    if (B <= 65535 && cluster_size_for(B, Hkv) > 0) return 1;
    return 2 + (with_append ? 1 : 0);
}

size_t paged_gqa_workspace_bytes_impl(int B, int Hq, int Hkv, int D) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0) return 0;
    (void)Hkv;
    return (size_t)(kMaxGrid + B) * Hq * (D + 2) * sizeof(float);
}

int paged_gqa_decode_impl(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes, const void* k_scales,
                          const void* v_scales, const int32_t* block_table, const int32_t* lengths, void* out,
                          void* workspace, size_t workspace_bytes, int B, int Hq, int Hkv, int D, int page_size,
                          int64_t num_pages, int max_blocks, int group_size, float scale, int q_dtype,
                          int scale_dtype, int sink_tokens, int window_size, cudaStream_t stream) {
    int tp_in_slot = -1, tp_out_slot = -1;
    tp_take(&tp_in_slot, &tp_out_slot);
    if ((bits != 4 && bits != 8) || q == nullptr || k_codes == nullptr || v_codes == nullptr || k_scales == nullptr ||
        v_scales == nullptr || block_table == nullptr || lengths == nullptr || (out == nullptr && tp_out_slot < 0))
        return B200Q_ERR_BAD_ARG;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 ||
        group_size <= 0 || Hq % Hkv != 0 || !is_act_dtype(q_dtype) || !is_scale_dtype(scale_dtype) ||
        sink_tokens < 0 || window_size < 0)
        return B200Q_ERR_BAD_ARG;
    if (D > 128) return B200Q_ERR_UNSUPPORTED;
    const int Gd = (D + group_size - 1) / group_size;
    const int group = Hq / Hkv;
    const int dp = bits == 4 ? D / 2 : D;

    const bool fast_ok = tuning_get("attn.force_simple") == 0 && D == 128 && q_dtype == B200Q_F16 &&
                         scale_dtype == B200Q_F16 && (group_size == 32 || group_size == 64) && group <= 8 &&
                         Hkv <= kAttnWarps && page_size == 16 && B <= kMaxBatchFast &&
                         ((uintptr_t)q % 16 == 0) && ((uintptr_t)k_codes % 16 == 0) && ((uintptr_t)v_codes % 16 == 0) &&
                         ((uintptr_t)k_scales % 8 == 0) && ((uintptr_t)v_scales % 8 == 0);
    if (!fast_ok && tp_out_slot >= 0) return B200Q_ERR_UNSUPPORTED;   // the exchange exists only in the split-KV kernels
    if (!fast_ok) {
        SimpleParams sp = {q, k_codes, v_codes, k_scales, v_scales, block_table, lengths, out,
                           B, Hq, Hkv, D, page_size, max_blocks, group_size, Gd, bits, q_dtype, scale_dtype,
                           num_pages, scale, sink_tokens, window_size, nullptr, 0, 0, 0};
        const int warps = 4;
        paged_attn_simple_kernel<<<(B * Hq + warps - 1) / warps, warps * 32, 0, stream>>>(sp);
        return finish_launch();
    }
    // small batches: one cluster per (sequence, kv head), merged on chip - no workspace, no second launch
    const int cluster = window_size == 0 && B <= 65535 && Hkv <= 65535 ? cluster_size_for(B, Hkv) : 0;
    if (cluster > 0) {
        ClusterAttnParams c = {};
        if (tp_out_slot >= 0) c.tp_out = tp_slot(tp_out_slot)->out;
        c.q = (const __half*)q;
        c.k_codes = const_cast<uint8_t*>(k_codes); c.v_codes = const_cast<uint8_t*>(v_codes);
        c.k_scales = (__half*)const_cast<void*>(k_scales); c.v_scales = (__half*)const_cast<void*>(v_scales);
        c.block_table = block_table; c.lengths = lengths; c.out = out;
        c.B = B; c.Hq = Hq; c.Hkv = Hkv; c.P = page_size; c.max_blocks = max_blocks; c.G = group_size; c.Gd = Gd;
        c.group = group; c.bits = bits; c.S = cluster; c.num_pages = num_pages; c.scale = scale;
        c.row_bytes = Hkv * dp; c.scale_row_halves = Hkv * Gd;
        const int rc = launch_cluster_attention(c, stream);
        if (rc != B200Q_ERR_UNSUPPORTED) return rc;
    }
    if (workspace == nullptr || workspace_bytes < paged_gqa_workspace_bytes_impl(B, Hq, Hkv, D)) return B200Q_ERR_WORKSPACE;

    AttnParams p = {};
    if (tp_out_slot >= 0) p.tp_out = tp_slot(tp_out_slot)->out;
    p.q = (const __half*)q; p.k_codes = k_codes; p.v_codes = v_codes;
    p.k_scales = (const __half*)k_scales; p.v_scales = (const __half*)v_scales;
    p.block_table = block_table; p.lengths = lengths; p.partial = (float*)workspace; p.out = out;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.P = page_size; p.max_blocks = max_blocks; p.G = group_size; p.Gd = Gd;
    p.group = group; p.num_pages = num_pages; p.scale = scale; p.q_dtype = q_dtype; p.bits = bits;
    p.subs = subs_for(Hkv);
    p.sink = sink_tokens;
    p.window = window_size;
    p.row_bytes = Hkv * dp;
    p.scale_row_halves = Hkv * Gd;
    p.slot_bytes = (bits == 4 ? 2048 : 4096) + 256;
    int ctas_per_sm = tuning_get("attn.ctas_per_sm");
    if (ctas_per_sm <= 0) ctas_per_sm = B200Q_ATTN_CTAS;
    // At least three pages per range (by the block table's capacity; the lengths live on the device): short
    // batches otherwise pay for partial results and their merge more than for the KV bytes (measured on the
    // 32-layer stack at batch 1, context 4096: 2 -> 2.32-2.35, 3 -> 2.26, 4 -> 2.30, 8 -> 2.46 ms per step).
    const int64_t pages_cap = (int64_t)B * max_blocks;
    int min_pages = tuning_get("attn.min_pages");
    if (min_pages <= 0) min_pages = 3;
    p.grid = (int)std::max<int64_t>(1, std::min<int64_t>(std::min(kMaxGrid, sm_count() * ctas_per_sm),
                                                         (pages_cap + min_pages - 1) / min_pages));
    const int launch_grid = (p.grid + p.subs - 1) / p.subs;   // CTAs: each covers `subs` ranges
    const bool two = launch_grid > sm_count();
    const int stages = ring_depth(bits, two);

    uint32_t off = 0;
    p.off_prefix = off; off += align_up_u32((B + 1) * sizeof(int), 16);
    off = align_up_u32(off, 128);
    p.off_ring = off;
    const uint32_t cap = (uint32_t)max_smem_optin();
    if (off + (uint64_t)stages * kAttnWarps * p.slot_bytes > cap) return B200Q_ERR_UNSUPPORTED;
    p.stages = stages;
    const uint32_t total_smem = off + stages * kAttnWarps * p.slot_bytes;

    const bool g32 = group_size == 32;
    using KernelFn = void (*)(AttnParams);
    KernelFn kernel;
    if (two)
        kernel = bits == 4 ? (g32 ? paged_attn_kernel<4, 5, true> : paged_attn_kernel<4, 6, true>)
                           : (g32 ? paged_attn_kernel<8, 5, true> : paged_attn_kernel<8, 6, true>);
    else
        kernel = bits == 4 ? (g32 ? paged_attn_kernel<4, 5, false> : paged_attn_kernel<4, 6, false>)
                           : (g32 ? paged_attn_kernel<8, 5, false> : paged_attn_kernel<8, 6, false>);
    static bool configured[2][2][2][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[two][bits == 4][g32][dev & 63]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap) != cudaSuccess)
            return B200Q_ERR_LAUNCH;
        configured[two][bits == 4][g32][dev & 63] = true;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(launch_grid);
        cfg.blockDim = dim3(kAttnThreads);
        cfg.dynamicSmemBytes = total_smem;
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = tuning_get("no_pdl") ? 0 : 1;
        if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return B200Q_ERR_LAUNCH;
    }
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(B * Hq);
        const bool wide = B * Hq < 2 * sm_count();
        cfg.blockDim = dim3((wide ? 32 : 8) * 32);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = tuning_get("no_pdl") ? 0 : 1;
        if (cudaLaunchKernelEx(&cfg, wide ? paged_attn_merge_kernel<32> : paged_attn_merge_kernel<8>, p) != cudaSuccess)
            return B200Q_ERR_LAUNCH;
    }
    return finish_launch();
}

// Decode-layer attention in one call: split + rotate + append (as rope_kv_append_impl) followed by the attention over
// the cache including the new token.  Small batches run it as ONE launch of the cluster kernel; otherwise the two
// stages are launched one after the other (q_scratch [B, Hq, D] then holds the rotated queries).
int rope_kv_append_impl(const void* qkv, const float* cos_table, const float* sin_table, const int32_t* positions,
                        const int32_t* block_table, void* q_out, uint8_t* k_codes, uint8_t* v_codes, void* k_scales,
                        void* v_scales, int bits, int B, int Hq, int Hkv, int D, int page_size, int64_t num_pages,
                        int max_blocks, int group_size, int table_len, cudaStream_t stream);

int rope_append_attention_impl(const void* qkv, const float* cos_table, const float* sin_table, const int32_t* positions,
                               int table_len, int bits, uint8_t* k_codes, uint8_t* v_codes, void* k_scales, void* v_scales,
                               const int32_t* block_table, const int32_t* lengths, void* out, void* q_scratch, void* workspace,
                               size_t workspace_bytes, int B, int Hq, int Hkv, int D, int page_size, int64_t num_pages,
                               int max_blocks, int group_size, float scale, cudaStream_t stream) {
    if (qkv == nullptr || cos_table == nullptr || sin_table == nullptr || positions == nullptr || k_codes == nullptr ||
        v_codes == nullptr || k_scales == nullptr || v_scales == nullptr || block_table == nullptr || lengths == nullptr) {
        tp_discard();
        return B200Q_ERR_BAD_ARG;
    }
    if ((bits != 4 && bits != 8) || B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || page_size <= 0 || num_pages <= 0 ||
        max_blocks <= 0 || group_size <= 0 || table_len <= 0 || Hq % Hkv != 0) {
        tp_discard();
        return B200Q_ERR_BAD_ARG;
    }
    const int group = Hq / Hkv;
    const int Gd = (D + group_size - 1) / group_size;
    const int dp = bits == 4 ? D / 2 : D;
    const bool fast_ok = tuning_get("attn.force_simple") == 0 && D == 128 && (group_size == 32 || group_size == 64) &&
                         group <= 8 && Hkv <= kAttnWarps && page_size == 16 && B <= 65535 && ((uintptr_t)qkv % 16 == 0) &&
                         ((uintptr_t)k_codes % 16 == 0) && ((uintptr_t)v_codes % 16 == 0) && ((uintptr_t)k_scales % 8 == 0) &&
                         ((uintptr_t)v_scales % 8 == 0);
    const int cluster = fast_ok ? cluster_size_for(B, Hkv) : 0;
    if (cluster > 0) {
        int tp_in_slot = -1, tp_out_slot = -1;
        tp_take(&tp_in_slot, &tp_out_slot);
        if (out == nullptr && tp_out_slot < 0) return B200Q_ERR_BAD_ARG;
        ClusterAttnParams c = {};
        if (tp_out_slot >= 0) c.tp_out = tp_slot(tp_out_slot)->out;
        c.qkv = (const __half*)qkv; c.cos_table = cos_table; c.sin_table = sin_table; c.positions = positions;
        c.table_len = table_len; c.fused = 1;
        c.k_codes = k_codes; c.v_codes = v_codes; c.k_scales = (__half*)k_scales; c.v_scales = (__half*)v_scales;
        c.block_table = block_table; c.lengths = lengths; c.out = out;
        c.B = B; c.Hq = Hq; c.Hkv = Hkv; c.P = page_size; c.max_blocks = max_blocks; c.G = group_size; c.Gd = Gd;
        c.group = group; c.bits = bits; c.S = cluster; c.num_pages = num_pages; c.scale = scale;
        c.row_bytes = Hkv * dp; c.scale_row_halves = Hkv * Gd;
        const int rc = launch_cluster_attention(c, stream);
        if (rc != B200Q_ERR_UNSUPPORTED) return rc;
        if (q_scratch == nullptr) return B200Q_ERR_WORKSPACE;
        // fall through to the two-stage route with the exchange slots restored for the attention stage
        int rc2 = rope_kv_append_impl(qkv, cos_table, sin_table, positions, block_table, q_scratch, k_codes, v_codes, k_scales,
                                      v_scales, bits, B, Hq, Hkv, D, page_size, num_pages, max_blocks, group_size, table_len, stream);
        if (rc2 != B200Q_OK) return rc2;
        if (tp_out_slot >= 0) return B200Q_ERR_UNSUPPORTED;
        return paged_gqa_decode_impl(bits, q_scratch, k_codes, v_codes, k_scales, v_scales, block_table, lengths, out, workspace,
                                     workspace_bytes, B, Hq, Hkv, D, page_size, num_pages, max_blocks, group_size, scale,
                                     B200Q_F16, B200Q_F16, 0, 0, stream);
    }
    if (q_scratch == nullptr) {
        tp_discard();
        return B200Q_ERR_WORKSPACE;
    }
    const int rc = rope_kv_append_impl(qkv, cos_table, sin_table, positions, block_table, q_scratch, k_codes, v_codes, k_scales,
                                       v_scales, bits, B, Hq, Hkv, D, page_size, num_pages, max_blocks, group_size, table_len, stream);
    if (rc != B200Q_OK) {
        tp_discard();
        return rc;
    }
    return paged_gqa_decode_impl(bits, q_scratch, k_codes, v_codes, k_scales, v_scales, block_table, lengths, out, workspace,
                                 workspace_bytes, B, Hq, Hkv, D, page_size, num_pages, max_blocks, group_size, scale, B200Q_F16,
                                 B200Q_F16, 0, 0, stream);
}

// ------------------------------------------------------------------------------------------------
// Variant without a caller-supplied workspace: the split-KV partials live in a fixed array in
// device memory that belongs to the library image.
// ------------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 8u << 20;     // 8 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

size_t paged_gqa_static_scratch_bytes_impl() { return kStaticScratchBytes; }

int paged_gqa_decode_static_impl(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                                 const void* k_scales, const void* v_scales, const int32_t* block_table,
                                 const int32_t* lengths, void* out, int B, int Hq, int Hkv, int D, int page_size,
                                 int64_t num_pages, int max_blocks, int group_size, float scale, int q_dtype,
                                 int scale_dtype, cudaStream_t stream) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0) {
        tp_discard();
        return B200Q_ERR_BAD_ARG;
    }
    // In host code the array's name is only a handle; the device address has to be asked for, once per
    // device, with that device current.
    static void* scratch_ptr[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        tp_discard();
        return B200Q_ERR_LAUNCH;
    }
    void* ptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (scratch_ptr[dev] == nullptr) {
            void* p = nullptr;
            if (cudaGetSymbolAddress(&p, g_attn_static_scratch) != cudaSuccess || p == nullptr) {
                tp_discard();
                return B200Q_ERR_LAUNCH;
            }
            scratch_ptr[dev] = p;
        }
        ptr = scratch_ptr[dev];
    }
    // Only the split-KV kernels use the scratch: the size check is theirs (problems that take the one-warp-per-head
    // kernel need none), reported here under this entry point's own code.
    const int rc = paged_gqa_decode_impl(bits, q, k_codes, v_codes, k_scales, v_scales, block_table, lengths, out, ptr,
                                         kStaticScratchBytes, B, Hq, Hkv, D, page_size, num_pages, max_blocks, group_size,
                                         scale, q_dtype, scale_dtype, 0, 0, stream);
    return rc == B200Q_ERR_WORKSPACE ? B200Q_ERR_STATIC_SCRATCH : rc;
}

// ------------------------------------------------------------------------------------------------
// Block-sparse decode: key j of a sequence of L tokens is attended iff block_mask[(L-1)/bs][j/bs] != 0 (the decode
// row of the reference's block_sparse mask; the causal bound j <= L-1 holds for every cached token).
// When bs is a multiple of the page size the attended keys are whole pages (and possibly the partly filled last
// one), and softmax attention does not depend on the order of its keys: one warp per sequence compacts the
// attended pages into a private block table with the matching length, and the dense kernels run on that.
// ------------------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(128) block_sparse_pages_kernel(const int32_t* block_table, const int32_t* lengths,
                                                                 const uint8_t* block_mask, int n_qblocks, int n_kblocks,
                                                                 int pages_per_block, int P, int max_blocks, int B,
                                                                 int32_t* table_out, int32_t* lengths_out) {
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= B) return;
    const int L = clamp_len(lengths[b], max_blocks * P);
    const int npages = (L + P - 1) / P;
    const int bs = pages_per_block * P;
    const int qb = L > 0 ? (L - 1) / bs : 0;
    const uint8_t* row = (L > 0 && qb < n_qblocks) ? block_mask + (size_t)qb * n_kblocks : nullptr;
    const int32_t* src = block_table + (size_t)b * max_blocks;
    int32_t* dst = table_out + (size_t)b * max_blocks;
    int count = 0, tokens = 0;
    for (int p0 = 0; p0 < npages; p0 += 32) {
        const int pg = p0 + lane;
        bool vis = false;
        if (pg < npages && row != nullptr) {
            const int kb = pg / pages_per_block;
            vis = kb < n_kblocks && row[kb] != 0;
        }
        const uint32_t ballot = __ballot_sync(0xffffffffu, vis);
        if (vis) dst[count + __popc(ballot & ((1u << lane) - 1u))] = src[pg];
        count += __popc(ballot);
        // every attended page is full except the sequence's last page
        tokens += __popc(ballot) * P;
        if (npages - 1 >= p0 && npages - 1 < p0 + 32 && ((ballot >> (npages - 1 - p0)) & 1u)) tokens -= npages * P - L;
    }
    for (int i = count + lane; i < max_blocks; i += 32) dst[i] = -1;
    if (lane == 0) lengths_out[b] = tokens;
}
}  // namespace

int paged_gqa_decode_block_sparse_impl(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                                       const void* k_scales, const void* v_scales, const int32_t* block_table,
                                       const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes,
                                       const uint8_t* block_mask, int n_qblocks, int n_kblocks, int block_size,
                                       int32_t* page_scratch, int B, int Hq, int Hkv, int D, int page_size,
                                       int64_t num_pages, int max_blocks, int group_size, float scale, int q_dtype,
                                       int scale_dtype, cudaStream_t stream) {
    if (block_mask == nullptr || n_qblocks <= 0 || n_kblocks <= 0 || block_size <= 0) {
        tp_discard();
        return B200Q_ERR_BAD_ARG;
    }
    if (page_scratch != nullptr && page_size > 0 && block_size % page_size == 0 && B > 0 && max_blocks > 0 &&
        block_table != nullptr && lengths != nullptr) {
        int32_t* table2 = page_scratch;
        int32_t* lengths2 = page_scratch + (size_t)B * max_blocks;
        block_sparse_pages_kernel<<<(B + 3) / 4, 128, 0, stream>>>(block_table, lengths, block_mask, n_qblocks, n_kblocks,
                                                                  block_size / page_size, page_size, max_blocks, B, table2,
                                                                  lengths2);
        const int rc = finish_launch();
        if (rc != B200Q_OK) {
            tp_discard();
            return rc;
        }
        return paged_gqa_decode_impl(bits, q, k_codes, v_codes, k_scales, v_scales, table2, lengths2, out, workspace,
                                     workspace_bytes, B, Hq, Hkv, D, page_size, num_pages, max_blocks, group_size, scale,
                                     q_dtype, scale_dtype, 0, 0, stream);
    }
    // any block size: the one-warp-per-head kernel with a per-token test
    tp_discard();
    if ((bits != 4 && bits != 8) || q == nullptr || k_codes == nullptr || v_codes == nullptr || k_scales == nullptr ||
        v_scales == nullptr || block_table == nullptr || lengths == nullptr || out == nullptr)
        return B200Q_ERR_BAD_ARG;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 ||
        group_size <= 0 || Hq % Hkv != 0 || !is_act_dtype(q_dtype) || !is_scale_dtype(scale_dtype))
        return B200Q_ERR_BAD_ARG;
    if (D > 128) return B200Q_ERR_UNSUPPORTED;
    SimpleParams sp = {q, k_codes, v_codes, k_scales, v_scales, block_table, lengths, out,
                       B, Hq, Hkv, D, page_size, max_blocks, group_size, (D + group_size - 1) / group_size, bits, q_dtype,
                       scale_dtype, num_pages, scale, 0, 0, block_mask, block_size, n_qblocks, n_kblocks};
    const int warps = 4;
    paged_attn_simple_kernel<<<(B * Hq + warps - 1) / warps, warps * 32, 0, stream>>>(sp);
    return finish_launch();
}

}  // namespace b200q
