// Quantized skinny GEMM for decode on the 5th-generation tensor cores (tcgen05, sm_100a):
//
//   y[b, n] = sum_k x[b, k] * (code[n, k] - zero[n, k/G]) * scale[n, k/G]          b < B <= 64
//
// The weights are the A operand and live in TENSOR MEMORY, the activations are the B operand in
// shared memory, the accumulator D[128 weight rows, batch columns] stays in tensor memory:
//
//   TMA (one elected thread)      2-D tiled copies, 128-byte swizzle: 128 rows x 128 bytes of codes per
//                                 stage and matrix, plus the rows' scales / zero points of the stage
//   dequantise warps (8)          thread = weight row.  Codes come out of shared memory 16 bytes at a time
//                                 (conflict-free through the swizzle), become fp16 weights in registers,
//                                     w = ((1024+q) - (1024+rint(z))) * s + (rint(z) - z) * s
//                                 (exact subtraction, then one fused multiply-add), and go to tensor memory
//                                 with tcgen05.st, 128 k (64 columns) per chunk.  No loop-carried dependency:
//                                 the work is a pure stream.
//   activation warps (2)          write the stage's activation rows (optionally x := rmsnorm(x + residual))
//                                 into shared memory in the K-major 128-byte-swizzled operand layout
//   MMA (one elected thread)      tcgen05.mma.kind::f16, M = 128, N = batch rounded up to 16, K = 16,
//                                 A from tensor memory, B through a shared-memory descriptor; tcgen05.commit
//                                 releases the chunk / the stage / the accumulator
//   epilogue (warps 0-3)          tcgen05.ld of D, clamp, round, residual add or SwiGLU, store
//
// A CTA owns row tiles of 128 rows.  When there are fewer tiles than SMs the K range of a tile is split
// over the CTAs of a thread-block cluster; the partial accumulators are summed in rank order through
// distributed shared memory by the cluster's first CTA (deterministic, no global scratch).
// Every wait is bounded; a wait that runs out records an event in the status word and the kernel
// carries on without the data so that it always terminates and frees its tensor memory.
#include "gemv_params.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <functional>
#include <mutex>
#include <unordered_map>

namespace b200q {

B200Q_DEFINE_STATUS_WORD(qgemm_ts_read_status)

namespace {

constexpr int kDeqWarps = 8;                   // two groups of four (one warp per 32-lane quarter of tensor memory)
constexpr int kTmaWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kXWarp0 = 10;
constexpr int kXWarps = 2;
constexpr int kTsThreads = (kDeqWarps + 2 + kXWarps) * 32;     // 384
constexpr int kRows = 128;                     // weight rows per tile = lanes of tensor memory
constexpr int kChunkK = 128;                   // k per chunk of A in tensor memory (64 columns of 2 halves)
constexpr int kChunkCols = kChunkK / 2;
constexpr int kRowBytes = 128;                 // bytes of one weight row per stage = the swizzle span
constexpr int kWTile = kRows * kRowBytes;      // 16 KB of codes per stage and matrix
constexpr int kMetaTile = kRows * 16;          // 2 KB: 8 fp16 scales (or zero points) per row
constexpr int kMaxStages = 6;
constexpr int kMaxASlots = 6;
constexpr uint32_t kTsWaitLimit = 1u << 20;

struct alignas(64) TsParams {
    CUtensorMap wmap[2];        // codes [N, row_bytes] u8, box 128 B x 128 rows, 128-byte swizzle
    CUtensorMap smap[2];        // scales [N, Gn] fp16 as bytes, box 16 B x 128 rows
    CUtensorMap zmap[2];        // zero points, same
    const __half* x;            // [B, K]
    const __half* res_in;       // norm prologue: rows = rmsnorm(x + res_in); may be null
    const void* norm_w;         // [K]; null = no prologue
    __half* z_out;              // [B, K] or null
    __half* normed_out;         // [B, K] or null
    const __half* residual;     // plain: out = cast(residual + cast(y)); may be null
    __half* y;
    __half* gate_out;
    __half* up_out;
    __half* act_out;
    float eps;
    int norm_w_dtype;
    int B, N, K;
    int has_z;
    int ncols;                  // MMA N: batch rows rounded up to a multiple of 16
    int tiles;                  // row tiles of 128
    int split;                  // CTAs per cluster = parts of the K range
    int n_stage_total;          // K / (k per stage)
    int stages;                 // ring depth
    int a_slots;                // chunks of A in tensor memory
    int a_col0;                 // first column of the A ring (the accumulators sit below it)
    int tmem_cols;              // columns allocated (power of two)
    uint32_t stage_bytes, off_meta, off_x;     // layout of one stage: [codes x MATS][scales, zeros x MATS][activations]
};

// ---- PTX wrappers specific to this kernel ---------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// D[128, N] (+)= A[128, 16] (tensor memory) * B[16, N] (shared memory, K-major)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
        "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
        "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t local_addr, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ uint32_t hadd2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t a, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, int event, bool& ok) {
    const bool got = mbar_wait_bounded(bar, parity, &g_device_status, event, ok ? kTsWaitLimit : 64u);
    ok = ok && got;
    return got;
}

// Per-group constants of the dequantisation, each duplicated into both halves of a register:
//   w = ((base + q) + c_base) * s + r,   c_base = -(base + zi),  zi = rint(z),  r = (zi - z) * s
struct GroupConst { uint32_t s2, r2, c1024, c64; };
__device__ __forceinline__ GroupConst group_const(uint32_t s_bits, uint32_t z_bits) {
    GroupConst c;
    c.s2 = (s_bits & 0xFFFFu) | (s_bits << 16);
    const uint32_t z2 = (z_bits & 0xFFFFu) | (z_bits << 16);
    const __half2 zi = h2rint(*reinterpret_cast<const __half2*>(&z2));
    const uint32_t zi2 = *reinterpret_cast<const uint32_t*>(&zi);
    c.r2 = hmul2_u32(hsub2_u32(zi2, z2), c.s2);
    c.c1024 = hsub2_u32(0xE400E400u, zi2);        // -1024 - zi (exact: integers below 2048)
    c.c64 = hsub2_u32(0xD400D400u, zi2);          // -64 - zi
    return c;
}

template <int BITS, int LOGG, int MATS>
__global__ void __launch_bounds__(kTsThreads, 1) qgemm_ts_kernel(const __grid_constant__ TsParams p) {
    constexpr int KS = kRowBytes * 8 / BITS;           // k per stage: 256 (q4) or 128 (q8)
    constexpr int SC = KS / kChunkK;                   // k-chunks per stage
    constexpr int APS = SC * MATS;                     // chunks of A per stage
    constexpr int G = 1 << LOGG;
    constexpr int GPC = kChunkK / G > 0 ? kChunkK / G : 1;   // groups per chunk (G = 128: one)
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const sbase = smem_raw + (base - smem_u32(smem_raw));

    uint64_t* bars = reinterpret_cast<uint64_t*>(sbase);
    uint64_t* full_w = bars;                            // [stages] codes + scales of the stage have landed
    uint64_t* full_x = full_w + kMaxStages;             // [stages] activation rows of the stage are written
    uint64_t* empty_w = full_x + kMaxStages;            // [stages] dequantise warps are done with the codes
    uint64_t* empty_x = empty_w + kMaxStages;           // [stages] the MMAs reading the activation rows are done
    uint64_t* a_full = empty_x + kMaxStages;            // [a_slots] a chunk of A is in tensor memory
    uint64_t* a_free = a_full + kMaxASlots;             // [a_slots] the MMAs reading the chunk are done
    uint64_t* d_full = a_free + kMaxASlots;             // the tile's accumulator is complete
    uint64_t* d_free = d_full + 1;                      // the epilogue has read the accumulator
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sbase + 512);
    float* inv_rms = reinterpret_cast<float*>(sbase + 576);      // [B <= 64]
    const uint32_t stage0 = base + 1024;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = p.split > 1 ? cluster_rank() : 0u;
    const int cluster_id = (int)blockIdx.x / p.split;
    const int n_clusters = (int)gridDim.x / p.split;
    const int st_lo = (int)((int64_t)p.n_stage_total * rank / p.split);
    const int st_hi = (int)((int64_t)p.n_stage_total * (rank + 1) / p.split);
    const int n_st = st_hi - st_lo;
    const int my_tiles = cluster_id < p.tiles ? (p.tiles - cluster_id + n_clusters - 1) / n_clusters : 0;
    const int NS = p.stages;
    const int NA = p.a_slots;
    const int ncols = p.ncols;
    const int B = p.B;

    // ---- set-up: barriers, tensor memory, zeroed activation tiles (rows >= B stay zero for good) ----
    if (threadIdx.x == 0) {
        for (int i = 0; i < NS; ++i) {
            mbar_init(&full_w[i], 1);
            mbar_init(&full_x[i], kXWarps);
            mbar_init(&empty_w[i], APS == 1 ? 4 : kDeqWarps);
            mbar_init(&empty_x[i], 1);
        }
        for (int i = 0; i < NA; ++i) {
            mbar_init(&a_full[i], 4);
            mbar_init(&a_free[i], 1);
        }
        mbar_init(d_full, 1);
        mbar_init(d_free, 4);
        mbar_fence_init();
    }
    if (warp == kTmaWarp) tmem_alloc(tmem_slot, (uint32_t)p.tmem_cols);
    {
        const uint32_t x_bytes = (uint32_t)ncols * KS * 2;
        for (int s = 0; s < NS; ++s)
            for (uint32_t o = threadIdx.x * 16u; o < x_bytes; o += kTsThreads * 16u)
                sts128(stage0 + s * p.stage_bytes + p.off_x + o, make_uint4(0u, 0u, 0u, 0u));
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    pdl_launch_dependents();

    // ================================ TMA producer ================================================
    if (warp == kTmaWarp) {
        if (lane == 0) {
            bool ok = true;
            uint32_t it = 0;
            const uint32_t tx = MATS * (kWTile + kMetaTile * (p.has_z ? 2 : 1));
            for (int ti = 0; ti < my_tiles; ++ti) {
                const int n0 = (cluster_id + ti * n_clusters) * kRows;
                for (int s = st_lo; s < st_hi; ++s, ++it) {
                    const int slot = it % NS;
                    wait_bar(&empty_w[slot], ((it / NS) & 1u) ^ 1u, EV_GEMV_EMPTY_WAIT, ok);
                    uint8_t* st = sbase + 1024 + (size_t)slot * p.stage_bytes;
                    mbar_arrive_expect_tx(&full_w[slot], tx);
                    const int gx = (((s * KS) >> LOGG) * 2) & ~15;          // byte column of the stage's scales
#pragma unroll
                    for (int m = 0; m < MATS; ++m) {
                        tma_load_2d(st + m * kWTile, &p.wmap[m], s * kRowBytes, n0, &full_w[slot]);
                        tma_load_2d(st + p.off_meta + m * 2 * kMetaTile, &p.smap[m], gx, n0, &full_w[slot]);
                        if (p.has_z)
                            tma_load_2d(st + p.off_meta + m * 2 * kMetaTile + kMetaTile, &p.zmap[m], gx, n0, &full_w[slot]);
                    }
                }
            }
        }
    }
    // ================================ MMA issuer ==================================================
    else if (warp == kMmaWarp) {
        if (lane == 0) {
            bool ok = true;
            const uint32_t idesc = (1u << 4) | ((uint32_t)(ncols >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
            // K-major, 128-byte swizzle, 8-row groups 1024 bytes apart, descriptor version 1
            const uint64_t desc_hi = ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61) | (1ull << 16);
            uint32_t it = 0, a = 0;
            for (int ti = 0; ti < my_tiles; ++ti) {
                if (ti > 0) wait_bar(d_free, (uint32_t)(ti - 1) & 1u, EV_GEMV_EMPTY_WAIT, ok);
                tc_fence_after();
                for (int sl = 0; sl < n_st; ++sl, ++it) {
                    const int slot = it % NS;
                    wait_bar(&full_x[slot], (it / NS) & 1u, EV_GEMV_FULL_WAIT, ok);
                    const uint32_t xb = stage0 + slot * p.stage_bytes + p.off_x;
#pragma unroll 1
                    for (int u = 0; u < APS; ++u, ++a) {
                        const int c = u / MATS, m = u % MATS;
                        const int t = a % NA;
                        wait_bar(&a_full[t], (a / NA) & 1u, EV_GEMV_FULL_WAIT, ok);
                        tc_fence_after();
                        const uint32_t a_t = tmem + (uint32_t)(p.a_col0 + t * kChunkCols);
                        const uint32_t d_t = tmem + (uint32_t)(m * ncols);
#pragma unroll
                        for (int i = 0; i < kChunkK / 16; ++i) {
                            const uint32_t xa = xb + (uint32_t)(c * 2 + (i >> 2)) * (uint32_t)(ncols * 128) + (i & 3) * 32;
                            const uint64_t desc = desc_hi | (uint64_t)((xa & 0x3FFFFu) >> 4);
                            tc_mma_ts(d_t, a_t + i * 8, desc, idesc, (sl == 0 && c == 0 && i == 0) ? 0u : 1u);
                        }
                        tc_commit(&a_free[t]);
                    }
                    tc_commit(&empty_x[slot]);
                }
                tc_commit(d_full);
            }
        }
    }
    // ================================ activation warps ============================================
    else if (warp >= kXWarp0) {
        pdl_wait();
        const int xt = threadIdx.x - kXWarp0 * 32;             // 0 .. 63
        const int xw = warp - kXWarp0;
        // rmsnorm prologue: one warp per batch row, fixed summation order
        if (p.norm_w != nullptr) {
            for (int b = xw; b < B; b += kXWarps) {
                float ss = 0.0f;
                for (int k = lane * 8; k < p.K; k += 256) {
                    const uint4 ux = *reinterpret_cast<const uint4*>(p.x + (size_t)b * p.K + k);
                    const __half2* hx = reinterpret_cast<const __half2*>(&ux);
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) { v[2 * i] = __low2float(hx[i]); v[2 * i + 1] = __high2float(hx[i]); }
                    if (p.res_in != nullptr) {
                        const uint4 ur = *reinterpret_cast<const uint4*>(p.res_in + (size_t)b * p.K + k);
                        const __half2* hr = reinterpret_cast<const __half2*>(&ur);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            v[2 * i] = __half2float(__float2half_rn(v[2 * i] + __low2float(hr[i])));
                            v[2 * i + 1] = __half2float(__float2half_rn(v[2 * i + 1] + __high2float(hr[i])));
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) inv_rms[b] = rsqrtf(ss / (float)p.K + p.eps);
            }
            named_bar_sync(1, kXWarps * 32);
        }
        bool ok = true;
        uint32_t it = 0;
        constexpr int PPR = KS / 8;                            // 16-byte pieces per batch row and stage
        const bool writes_side = cluster_id == 0;              // the cluster of tile 0 covers the whole K range
        for (int ti = 0; ti < my_tiles; ++ti) {
            for (int s = st_lo; s < st_hi; ++s, ++it) {
                const int slot = it % NS;
                wait_bar(&empty_x[slot], ((it / NS) & 1u) ^ 1u, EV_GEMV_EMPTY_WAIT, ok);
                const uint32_t xb = stage0 + slot * p.stage_bytes + p.off_x;
                const int k0 = s * KS;
                for (int idx = xt; idx < B * PPR; idx += kXWarps * 32) {
                    const int b = idx / PPR;
                    const int pc = idx - b * PPR;
                    const int k = k0 + pc * 8;
                    uint4 u = *reinterpret_cast<const uint4*>(p.x + (size_t)b * p.K + k);
                    if (p.norm_w != nullptr) {
                        const __half2* hx = reinterpret_cast<const __half2*>(&u);
                        float v[8];
#pragma unroll
                        for (int i = 0; i < 4; ++i) { v[2 * i] = __low2float(hx[i]); v[2 * i + 1] = __high2float(hx[i]); }
                        if (p.res_in != nullptr) {
                            const uint4 ur = *reinterpret_cast<const uint4*>(p.res_in + (size_t)b * p.K + k);
                            const __half2* hr = reinterpret_cast<const __half2*>(&ur);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                v[2 * i] = __half2float(__float2half_rn(v[2 * i] + __low2float(hr[i])));
                                v[2 * i + 1] = __half2float(__float2half_rn(v[2 * i + 1] + __high2float(hr[i])));
                            }
                        }
                        if (ti == 0 && writes_side && p.z_out != nullptr) {
                            __half2 zo[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) zo[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                            *reinterpret_cast<uint4*>(p.z_out + (size_t)b * p.K + k) = *reinterpret_cast<const uint4*>(zo);
                        }
                        const float inv = inv_rms[b];
                        __half2 no[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float w0 = load_as_f32(p.norm_w, p.norm_w_dtype, k + 2 * i);
                            const float w1 = load_as_f32(p.norm_w, p.norm_w_dtype, k + 2 * i + 1);
                            no[i] = __floats2half2_rn(v[2 * i] * inv * w0, v[2 * i + 1] * inv * w1);
                        }
                        u = *reinterpret_cast<const uint4*>(no);
                        if (ti == 0 && writes_side && p.normed_out != nullptr)
                            *reinterpret_cast<uint4*>(p.normed_out + (size_t)b * p.K + k) = u;
                    }
                    if (BITS == 4) {
                        // the order in which the dequantise warps emit the 8 codes of a 32-bit word: (0,4) (1,5) (2,6) (3,7)
                        u = make_uint4(prmt(u.x, u.z, 0x5410), prmt(u.x, u.z, 0x7632), prmt(u.y, u.w, 0x5410),
                                       prmt(u.y, u.w, 0x7632));
                    }
                    const uint32_t dst = xb + (uint32_t)(pc >> 3) * (uint32_t)(ncols * 128) + (uint32_t)(b >> 3) * 1024u +
                                         (uint32_t)(b & 7) * 128u + (uint32_t)(((pc & 7) ^ (b & 7)) << 4);
                    sts128(dst, u);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_x[slot]);
            }
        }
    }
    // ================================ dequantise warps (+ epilogue on warps 0-3) ===================
    else {
        const int grp = warp >> 2;                             // chunks a with a % 2 == grp
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                     // weight row inside the tile = lane of tensor memory
        const uint32_t sw = (uint32_t)(r & 7);
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        bool ok = true;
        bool waited_pdl = false;
        uint32_t it = 0;
        for (int ti = 0; ti < my_tiles; ++ti) {
            const int n0 = (cluster_id + ti * n_clusters) * kRows;
            for (int s = st_lo; s < st_hi; ++s, ++it) {
                const int slot = it % NS;
                const bool mine = APS == 1 ? ((it & 1u) == (uint32_t)grp) : true;
                if (mine) {
                    wait_bar(&full_w[slot], (it / NS) & 1u, EV_GEMV_FULL_WAIT, ok);
                    const uint32_t st = stage0 + slot * p.stage_bytes;
#pragma unroll 1
                    for (int u = (APS == 1 ? 0 : grp); u < APS; u += 2) {
                        const uint32_t a = it * APS + u;
                        const int c = u / MATS, m = u % MATS;
                        const int t = a % NA;
                        wait_bar(&a_free[t], ((a / NA) & 1u) ^ 1u, EV_GEMV_EMPTY_WAIT, ok);
                        tc_fence_after();
                        const uint32_t wrow = st + m * kWTile + (uint32_t)r * kRowBytes;
                        const uint32_t mrow = st + p.off_meta + m * 2 * kMetaTile + (uint32_t)r * 16;
                        const int g0 = ((s * KS + c * kChunkK) >> LOGG) & 7;      // first group of the chunk inside the scale tile
                        // scales / zero points of the chunk's groups (1, 2 or 4 halves)
                        uint32_t sreg[2] = {0u, 0u}, zreg[2] = {0u, 0u};
                        if (LOGG == 5) {
                            sreg[0] = lds32(mrow + g0 * 2); sreg[1] = lds32(mrow + g0 * 2 + 4);
                            if (p.has_z) { zreg[0] = lds32(mrow + kMetaTile + g0 * 2); zreg[1] = lds32(mrow + kMetaTile + g0 * 2 + 4); }
                        } else {
                            const uint32_t sa = lds32(mrow + ((g0 * 2) & ~3));
                            sreg[0] = (LOGG == 7 && (g0 & 1)) ? sa >> 16 : sa;
                            if (p.has_z) {
                                const uint32_t za = lds32(mrow + kMetaTile + ((g0 * 2) & ~3));
                                zreg[0] = (LOGG == 7 && (g0 & 1)) ? za >> 16 : za;
                            }
                        }
                        const uint32_t a_t = lane_addr + (uint32_t)(p.a_col0 + t * kChunkCols);
#pragma unroll
                        for (int hb = 0; hb < 2; ++hb) {            // halves of the chunk: 64 k -> 32 columns
                            uint32_t out[32];
#pragma unroll
                            for (int sb = 0; sb < 2; ++sb) {        // 32 k -> 16 columns
                                const int k32 = hb * 2 + sb;        // 32-k block of the chunk
                                const int gi = (k32 * 32) >> LOGG;  // group of the chunk (0 for G = 128)
                                const uint32_t sbits = (gi & 1) ? sreg[gi >> 1] >> 16 : sreg[gi >> 1];
                                const uint32_t zbits = (gi & 1) ? zreg[gi >> 1] >> 16 : zreg[gi >> 1];
                                const GroupConst gc = group_const(sbits & 0xFFFFu, zbits & 0xFFFFu);
                                if (BITS == 4) {
                                    const uint4 v = lds128(wrow + ((((uint32_t)(c * 4 + k32)) ^ sw) << 4));
                                    const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                                    for (int w = 0; w < 4; ++w) {
                                        const uint32_t lo = w4[w], hi = w4[w] >> 8;
                                        out[sb * 16 + 4 * w + 0] = hfma2_u32(hadd2_u32(lop3_and_or(lo, 0x000F000Fu, 0x64006400u), gc.c1024), gc.s2, gc.r2);
                                        out[sb * 16 + 4 * w + 1] = hfma2_u32(hadd2_u32(lop3_and_or(lo, 0x00F000F0u, 0x54005400u), gc.c64), gc.s2, gc.r2);
                                        out[sb * 16 + 4 * w + 2] = hfma2_u32(hadd2_u32(lop3_and_or(hi, 0x000F000Fu, 0x64006400u), gc.c1024), gc.s2, gc.r2);
                                        out[sb * 16 + 4 * w + 3] = hfma2_u32(hadd2_u32(lop3_and_or(hi, 0x00F000F0u, 0x54005400u), gc.c64), gc.s2, gc.r2);
                                    }
                                } else {
#pragma unroll
                                    for (int q16 = 0; q16 < 2; ++q16) {
                                        const uint4 v = lds128(wrow + ((((uint32_t)(k32 * 2 + q16)) ^ sw) << 4));
                                        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                                        for (int w = 0; w < 4; ++w) {
                                            out[sb * 16 + q16 * 8 + 2 * w] = hfma2_u32(hadd2_u32(prmt(w4[w], 0x64646464u, 0x4140u), gc.c1024), gc.s2, gc.r2);
                                            out[sb * 16 + q16 * 8 + 2 * w + 1] = hfma2_u32(hadd2_u32(prmt(w4[w], 0x64646464u, 0x4342u), gc.c1024), gc.s2, gc.r2);
                                        }
                                    }
                                }
                            }
                            tc_st32(a_t + hb * 32, out);
                        }
                        tc_wait_st();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&a_full[t]);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty_w[slot]);
                }
            }
            // ---- epilogue of the tile (split == 1; with a split K range it follows the cluster exchange below) ----
            if (warp < 4 && p.split == 1) {
                if (!waited_pdl) { pdl_wait(); waited_pdl = true; }
                wait_bar(d_full, (uint32_t)ti & 1u, EV_GEMV_FULL_WAIT, ok);
                tc_fence_after();
                const int n = n0 + r;
                for (int c0 = 0; c0 < ncols; c0 += 16) {
                    float acc[MATS][16];
#pragma unroll
                    for (int m = 0; m < MATS; ++m) tc_ld16(lane_addr + (uint32_t)(m * ncols + c0), acc[m]);
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int b = c0 + j;
                            if (b >= B) break;
                            const size_t o = (size_t)b * p.N + n;
                            const float v0 = __half2float(__float2half_rn(fminf(fmaxf(acc[0][j], -65504.0f), 65504.0f)));
                            if (MATS == 1) {
                                float v = v0;
                                if (p.residual != nullptr) v = __half2float(p.residual[o]) + v;
                                p.y[o] = __float2half_rn(v);
                            } else {
                                const float v1 = __half2float(__float2half_rn(fminf(fmaxf(acc[MATS - 1][j], -65504.0f), 65504.0f)));
                                if (p.gate_out != nullptr) p.gate_out[o] = __float2half_rn(v0);
                                if (p.up_out != nullptr) p.up_out[o] = __float2half_rn(v1);
                                if (p.act_out != nullptr) p.act_out[o] = __float2half_rn((v0 / (1.0f + expf(-v0))) * v1);
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(d_free);
            }
        }
    }

    // ---- split K range: sum the partial accumulators of the cluster in rank order (one tile per cluster) ----
    if (p.split > 1) {
        __syncwarp();
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        const int dcols = MATS * ncols;
        bool ok = true;
        if (warp < 4 && my_tiles > 0) {
            wait_bar(d_full, 0u, EV_GEMV_FULL_WAIT, ok);
            tc_fence_after();
        }
        cluster_sync_all();          // every CTA of the cluster is done with its ring: the first CTA's ring is free
        if (warp < 4 && rank != 0 && my_tiles > 0) {
            for (int c0 = 0; c0 < dcols; c0 += 16) {
                float acc[16];
                tc_ld16(lane_addr + (uint32_t)c0, acc);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    st_cluster_f32(stage0 + (uint32_t)((((rank - 1) * dcols + c0 + j) * kRows + r) * 4), 0u, acc[j]);
            }
        }
        cluster_sync_all();          // the partial sums are in the first CTA's shared memory
        if (warp < 4 && rank == 0 && my_tiles > 0) {
            pdl_wait();
            const int n = cluster_id * kRows + r;
            const float* red = reinterpret_cast<const float*>(sbase + 1024);
            for (int c0 = 0; c0 < ncols; c0 += 16) {
                float acc[MATS][16];
#pragma unroll
                for (int m = 0; m < MATS; ++m) {
                    tc_ld16(lane_addr + (uint32_t)(m * ncols + c0), acc[m]);
                    for (int q = 1; q < p.split; ++q)
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[m][j] += red[(((q - 1) * dcols + m * ncols + c0 + j) * kRows + r)];
                }
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int b = c0 + j;
                        if (b >= B) break;
                        const size_t o = (size_t)b * p.N + n;
                        const float v0 = __half2float(__float2half_rn(fminf(fmaxf(acc[0][j], -65504.0f), 65504.0f)));
                        if (MATS == 1) {
                            float v = v0;
                            if (p.residual != nullptr) v = __half2float(p.residual[o]) + v;
                            p.y[o] = __float2half_rn(v);
                        } else {
                            const float v1 = __half2float(__float2half_rn(fminf(fmaxf(acc[MATS - 1][j], -65504.0f), 65504.0f)));
                            if (p.gate_out != nullptr) p.gate_out[o] = __float2half_rn(v0);
                            if (p.up_out != nullptr) p.up_out[o] = __float2half_rn(v1);
                            if (p.act_out != nullptr) p.act_out[o] = __float2half_rn((v0 / (1.0f + expf(-v0))) * v1);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kTmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, (uint32_t)p.tmem_cols);
    }
}

// ---- host side ---------------------------------------------------------------------------------------------------
struct MapKey {
    const void* ptr; uint64_t d0, d1; uint32_t b0, b1; int swz;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && b0 == o.b0 && b1 == o.b1 && swz == o.swz; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h = h * 1000003u ^ std::hash<uint64_t>()(k.d0 * 31 + k.d1);
        h = h * 1000003u ^ std::hash<uint64_t>()(((uint64_t)k.b0 << 32) | (k.b1 * 2 + k.swz));
        return h;
    }
};
std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

// 2-D byte tensor [d1 rows, d0 bytes] (rows d0 bytes apart), box b0 x b1.  The driver entry point is looked up at run
// time, so the library has no link-time dependency on libcuda.
bool tensor_map_2d(const void* ptr, uint64_t d0, uint64_t d1, uint32_t b0, uint32_t b1, bool swizzle128, CUtensorMap* out) {
    const MapKey key = {ptr, d0, d1, b0, b1, swizzle128 ? 1 : 0};
    std::lock_guard<std::mutex> lock(g_map_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return true; }
    if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || fn == nullptr)
            return false;
        g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }
    const cuuint64_t dims[2] = {d0, d1};
    const cuuint64_t strides[1] = {d0};
    const cuuint32_t box[2] = {b0, b1};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    const CUresult rc = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return false;
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, m);
    *out = m;
    return true;
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int BITS, int LOGG, int MATS>
int launch_ts(TsParams& p, cudaStream_t stream) {
    constexpr int KS = kRowBytes * 8 / BITS;
    const int sms = sm_count();
    p.n_stage_total = p.K / KS;
    p.tiles = (p.N + kRows - 1) / kRows;
    p.off_meta = MATS * kWTile;
    p.off_x = p.off_meta + MATS * 2 * kMetaTile;
    p.stage_bytes = p.off_x + (uint32_t)p.ncols * KS * 2;
    p.stage_bytes = (p.stage_bytes + 1023u) & ~1023u;
    // two kernels of a dependent chain can be resident on an SM together when each stays below half of its shared
    // memory; large batches take the whole SM
    const uint32_t cap = (uint32_t)max_smem_optin();
    uint32_t budget = p.ncols <= 16 ? std::min<uint32_t>(cap, 112u * 1024u) : cap;
    const int forced = tuning_get("ts.smem_kb");
    if (forced > 0) budget = std::min<uint32_t>(cap, (uint32_t)forced * 1024u);
    int stages = (int)((budget - 2048u) / p.stage_bytes);
    const int want = tuning_get("ts.stages");
    if (want > 0) stages = std::min(stages, want);
    stages = std::min(stages, kMaxStages);
    if (stages < 2) return B200Q_ERR_UNSUPPORTED;
    p.stages = stages;
    // tensor memory: accumulators below, ring of A chunks above
    const int dcols = MATS * p.ncols;
    p.a_col0 = std::max(32, (dcols + 31) / 32 * 32);
    p.tmem_cols = (p.a_col0 + 3 * kChunkCols <= 256) ? 256 : 512;
    p.a_slots = std::min(kMaxASlots, (p.tmem_cols - p.a_col0) / kChunkCols);
    if (p.a_slots < 2) return B200Q_ERR_UNSUPPORTED;
    // K split over a cluster when the tiles do not fill the SMs
    int split = 1;
    if (p.tiles < sms) split = std::min(8, sms / p.tiles);
    split = std::max(1, std::min(split, p.n_stage_total / 2));
    while (split > 1 && (uint64_t)(split - 1) * dcols * kRows * 4 > (uint64_t)stages * p.stage_bytes) --split;
    const int fs = tuning_get("ts.split");
    if (fs > 0) split = std::max(1, std::min({fs, 8, p.n_stage_total}));
    p.split = split;
    const int clusters = split > 1 ? p.tiles : std::min(p.tiles, sms);
    const uint32_t smem = 1024u + 1024u + (uint32_t)stages * p.stage_bytes;

    auto kernel = qgemm_ts_kernel<BITS, LOGG, MATS>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap) != cudaSuccess)
            return B200Q_ERR_LAUNCH;
        configured[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(clusters * split);
    cfg.blockDim = dim3(kTsThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (!tuning_get("no_pdl")) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (split > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = split;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return B200Q_ERR_LAUNCH;
    return finish_launch();
}

template <int BITS>
int dispatch_ts(TsParams& p, int G, bool gate_up, cudaStream_t stream) {
    if (gate_up) {
        if (G == 32) return launch_ts<BITS, 5, 2>(p, stream);
        if (G == 64) return launch_ts<BITS, 6, 2>(p, stream);
        return launch_ts<BITS, 7, 2>(p, stream);
    }
    if (G == 32) return launch_ts<BITS, 5, 1>(p, stream);
    if (G == 64) return launch_ts<BITS, 6, 1>(p, stream);
    return launch_ts<BITS, 7, 1>(p, stream);
}

}  // namespace

// Returns B200Q_ERR_UNSUPPORTED when the problem is outside this kernel (the caller then uses the other kernels).
int qgemm_ts(int bits, const GemvParams& g, bool gate_up, cudaStream_t stream) {
    if (g.act_dtype != B200Q_F16 || g.scale_dtype != B200Q_F16) return B200Q_ERR_UNSUPPORTED;
    if (g.G != 32 && g.G != 64 && g.G != 128) return B200Q_ERR_UNSUPPORTED;
    const int KS = kRowBytes * 8 / bits;
    if (g.K % KS != 0 || g.K % g.G != 0 || g.Gn % 8 != 0 || g.row_bytes % 16 != 0) return B200Q_ERR_UNSUPPORTED;
    if (g.B > 64 || g.tp_in.world > 0 || g.tp_out.world > 0) return B200Q_ERR_UNSUPPORTED;
    const int mats = gate_up ? 2 : 1;
    for (int m = 0; m < mats; ++m)
        if (!al16(g.w[m]) || !al16(g.s[m]) || (g.z[m] != nullptr && !al16(g.z[m]))) return B200Q_ERR_UNSUPPORTED;
    if (gate_up && ((g.z[0] == nullptr) != (g.z[1] == nullptr))) return B200Q_ERR_UNSUPPORTED;
    if (!al16(g.x) || (g.res_in != nullptr && !al16(g.res_in)) || (g.z_out != nullptr && !al16(g.z_out)) ||
        (g.normed_out != nullptr && !al16(g.normed_out)))
        return B200Q_ERR_UNSUPPORTED;
    if (g.K % 8 != 0) return B200Q_ERR_UNSUPPORTED;

    TsParams p = {};
    for (int m = 0; m < mats; ++m) {
        if (!tensor_map_2d(g.w[m], (uint64_t)g.row_bytes, (uint64_t)g.N, kRowBytes, kRows, true, &p.wmap[m])) return B200Q_ERR_UNSUPPORTED;
        if (!tensor_map_2d(g.s[m], (uint64_t)g.Gn * 2, (uint64_t)g.N, 16, kRows, false, &p.smap[m])) return B200Q_ERR_UNSUPPORTED;
        if (g.z[m] != nullptr &&
            !tensor_map_2d(g.z[m], (uint64_t)g.Gn * 2, (uint64_t)g.N, 16, kRows, false, &p.zmap[m]))
            return B200Q_ERR_UNSUPPORTED;
    }
    p.x = (const __half*)g.x; p.res_in = (const __half*)g.res_in; p.norm_w = g.norm_w; p.norm_w_dtype = g.norm_w_dtype;
    p.z_out = (__half*)g.z_out; p.normed_out = (__half*)g.normed_out; p.residual = (const __half*)g.residual;
    p.y = (__half*)g.y; p.gate_out = (__half*)g.gate_out; p.up_out = (__half*)g.up_out; p.act_out = (__half*)g.act_out;
    p.eps = g.eps; p.B = g.B; p.N = g.N; p.K = g.K; p.has_z = g.z[0] != nullptr ? 1 : 0;
    p.ncols = (g.B + 15) / 16 * 16;
    return bits == 4 ? dispatch_ts<4>(p, g.G, gate_up, stream) : dispatch_ts<8>(p, g.G, gate_up, stream);
}

}  // namespace b200q
