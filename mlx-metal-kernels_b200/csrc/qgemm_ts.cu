// Quantized skinny GEMM for decode on the 5th-generation tensor cores (tcgen05, sm_100a):
//
//   y[b, n] = sum_k x[b, k] * (code[n, k] - zero[n, k/G]) * scale[n, k/G]          b < B <= 32 per launch
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
//   activation warps (2 or 4)     each owns every n-th stage: one TMA copy per 64 k lands the stage's rows in the
//                                 operand tile (the copy's 128-byte swizzle is the K-major operand layout), then
//                                 the warp rewrites them in place where needed (order of the q4 codes inside a
//                                 32-bit word, x := rmsnorm(x + residual))
//   MMA (one warp, one elected    tcgen05.mma.kind::f16, M = 128, N = batch rounded up to 16, K = 16, A from
//        lane issues)             tensor memory, B through a shared-memory descriptor; tcgen05.commit releases
//                                 the chunk / the operand tile / the accumulator
//   epilogue (warps 0-3)          tcgen05.ld of D, clamp, round, residual add or SwiGLU, store
//
// Measured on B200: one tcgen05.mma of this shape occupies the tensor pipe for about 86 cycles whatever N <= 128,
// i.e. 128 rows x 16 k of weights per 86 cycles and SM.  That bounds q4 at about half of the HBM rate and q8 at
// about the full rate, for every batch up to 128 rows alike; the mma.sync kernel (gemv_fast.cuh) stays ahead for
// batches of a few rows.
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

constexpr int kRows = 128;                     // weight rows per tile = lanes of tensor memory
constexpr int kChunkK = 128;                   // k per chunk of A in tensor memory (64 columns of 2 halves)
constexpr int kChunkCols = kChunkK / 2;
constexpr int kRowBytes = 128;                 // bytes of one weight row per stage = the swizzle span
constexpr int kWTile = kRows * kRowBytes;      // 16 KB of codes per stage and matrix
constexpr int kMetaTile = kRows * 16;          // 2 KB: 8 fp16 scales (or zero points) per row
constexpr int kMaxStages = 8;
constexpr int kMaxASlots = 8;
constexpr int kMaxXTiles = 6;
constexpr uint32_t kTsWaitLimit = 1u << 20;
// Warp roles: [0, 8) dequantise (two groups of four: one warp per 32-lane quarter of tensor memory), 8 the TMA
// producer (also owns the tensor-memory allocation), 9 the MMA issuer, then the activation warps.  Two shapes:
// the compact one (2 activation warps) stays below half of an SM's shared memory, registers and tensor memory, so
// that two kernels of a dependent chain can be resident together; the whole-SM one (4 activation warps, deeper
// rings, all of tensor memory) is for large matrices (16 MB of codes and up) and for whatever the compact one cannot hold.
constexpr int kDeqWarps = 8;
constexpr int ts_xwarps(bool whole) { return whole ? 4 : 2; }
constexpr int ts_threads(bool whole) { return (kDeqWarps + 2 + ts_xwarps(whole)) * 32; }

struct alignas(64) TsParams {
    CUtensorMap wmap[2];        // codes [N, row_bytes] u8, box 128 B x 128 rows, 128-byte swizzle
    CUtensorMap smap[2];        // scales [N, Gn] fp16 as bytes, box 16 B x 128 rows
    CUtensorMap zmap[2];        // zero points, same
    CUtensorMap xmap;           // activations [B, K] fp16 as bytes, box 128 B (64 k) x B rows, 128-byte swizzle (= the operand layout)
    CUtensorMap rmap;           // residual rows of the norm prologue, box 64 k x B rows, no swizzle
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
    int stages;                 // depth of the ring of weight stages
    int a_slots;                // chunks of A in tensor memory
    int a_col0;                 // first column of the A ring (the accumulators sit below it)
    int tmem_cols;              // columns allocated (power of two)
    int x_tiles;                // depth of the ring of activation operand tiles
    uint32_t stage_bytes;       // one weight stage: [codes x MATS][scales, zeros x MATS]
    uint32_t off_meta;          // scales inside a stage
    uint32_t off_xt, xt_bytes;  // ring of operand tiles [ncols rows, k of a stage], K-major, 128-byte swizzle
    uint32_t off_res, res_bytes;  // residual rows of the norm prologue, one slot per operand tile (16-byte pieces, compact)
    uint32_t off_red;           // dedicated buffer for the cluster's partial sums (0: the weight ring is reused instead)
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
// Both are executed by the whole (converged) MMA warp; one elected lane issues.  Keeping the warp converged lets the
// compiler hold addresses and descriptors in uniform registers instead of moving them there before every instruction.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile(
        "{\n"
        ".reg .pred pe;\n"
        "elect.sync _|pe, 0xffffffff;\n"
        "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
        "}\n" ::"r"(smem_u32(bar))
        : "memory");
}
// D[128, N] (+)= A[128, 16] (tensor memory) * B[16, N] (shared memory, K-major)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p, pe;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "elect.sync _|pe, 0xffffffff;\n"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
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
__device__ __forceinline__ void arrive_remote(uint32_t local_bar_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_bar_addr), "r"(rank));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// bounded wait with cluster-scope acquire (the data guarded by the barrier was written by other CTAs of the cluster)
__device__ __forceinline__ bool wait_bar_cluster(uint64_t* bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
            "selp.b32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    atomicMax(&g_device_status, (int)EV_GEMV_FULL_WAIT);
    return false;
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

// The residual values of output row n for all batch columns, fetched before the accumulators are waited for and before
// the first store: y may alias the residual rows as far as the compiler knows, so a load placed after a store would
// wait for it - one global-memory latency per column.
template <int MATS>
__device__ __forceinline__ void ts_load_residual(const TsParams& p, int n, float (&res)[32]) {
    if (MATS == 1 && p.residual != nullptr && n < p.N) {
#pragma unroll
        for (int j = 0; j < 32; ++j) res[j] = j < p.B ? __half2float(p.residual[(size_t)j * p.N + n]) : 0.0f;
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) res[j] = 0.0f;
    }
}
// The epilogue of one 16-column slice: clamp, round, residual add or SwiGLU, store.
template <int MATS, int C0>
__device__ __forceinline__ void ts_store_cols(const TsParams& p, const float (&acc)[MATS][16], int n, const float (&res)[32]) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int b = C0 + j;
        if (b >= p.B) break;
        const size_t o = (size_t)b * p.N + n;
        const float v0 = __half2float(__float2half_rn(fminf(fmaxf(acc[0][j], -65504.0f), 65504.0f)));
        if (MATS == 1) {
            float v = v0;
            if (p.residual != nullptr) v = res[C0 + j] + v;
            p.y[o] = __float2half_rn(v);
        } else {
            const float v1 = __half2float(__float2half_rn(fminf(fmaxf(acc[MATS - 1][j], -65504.0f), 65504.0f)));
            if (p.gate_out != nullptr) p.gate_out[o] = __float2half_rn(v0);
            if (p.up_out != nullptr) p.up_out[o] = __float2half_rn(v1);
            if (p.act_out != nullptr) p.act_out[o] = __float2half_rn((v0 / (1.0f + expf(-v0))) * v1);
        }
    }
}

// Sum of squares of rmsnorm's input row z = cast(x + residual) for batch row b, by one warp; fixed summation order
// (lane-strided, then a butterfly), so every CTA and every launch shape gets the same bits.
__device__ __forceinline__ float row_inv_rms(const TsParams& p, int b, int lane) {
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
    return rsqrtf(ss / (float)p.K + p.eps);
}

template <int BITS, int LOGG, int MATS, bool WHOLE>
__global__ void __launch_bounds__(ts_threads(WHOLE), WHOLE ? 1 : 2) qgemm_ts_kernel(const __grid_constant__ TsParams p) {
    constexpr int DW = kDeqWarps;
    constexpr int kXWarps = ts_xwarps(WHOLE);
    constexpr int KS = kRowBytes * 8 / BITS;           // k per stage: 256 (q4) or 128 (q8)
    constexpr int SC = KS / kChunkK;                   // k-chunks per stage
    constexpr int APS = SC * MATS;                     // chunks of A per stage
    constexpr int NG = DW / 4;                         // dequantise groups; chunk a belongs to group a % NG
    constexpr int kTmaWarp = DW, kMmaWarp = DW + 1, kXWarp0 = DW + 2;
    constexpr int kThreads = ts_threads(WHOLE);
    constexpr int GPS = APS < NG ? APS : NG;           // groups that touch one stage
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const sbase = smem_raw + (base - smem_u32(smem_raw));

    uint64_t* bars = reinterpret_cast<uint64_t*>(sbase);
    uint64_t* full_w = bars;                            // [stages] codes + scales of the stage have landed
    uint64_t* empty_w = full_w + kMaxStages;            // [stages] dequantise warps are done with the codes
    uint64_t* full_x = empty_w + kMaxStages;            // [x_tiles] the operand tile of a stage is written
    uint64_t* empty_x = full_x + kMaxXTiles;            // [x_tiles] the MMAs reading the tile are done
    uint64_t* x_tma = empty_x + kMaxXTiles;             // [x_tiles] the raw activation rows of a stage have landed
    uint64_t* a_full = x_tma + kMaxXTiles;              // [a_slots] a chunk of A is in tensor memory
    uint64_t* a_free = a_full + kMaxASlots;             // [a_slots] the MMAs reading the chunk are done
    uint64_t* d_full = a_free + kMaxASlots;             // the tile's accumulator is complete
    uint64_t* d_free = d_full + 1;                      // the epilogue has read the accumulator
    uint64_t* red_bar = d_free + 1;                     // first CTA of a cluster: the other CTAs' partial sums have arrived
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sbase + 512);
    float* inv_rms = reinterpret_cast<float*>(sbase + 576);      // [B <= 64]
    const uint32_t stage0 = base + 1024;
    const uint32_t xt0 = base + p.off_xt;

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
    const int XT = p.x_tiles;
    const int ncols = p.ncols;
    const int B = p.B;

    // ---- set-up: barriers, tensor memory, zeroed operand tiles (rows >= B stay zero for good) ----
    if (threadIdx.x == 0) {
        for (int i = 0; i < NS; ++i) {
            mbar_init(&full_w[i], 1);
            mbar_init(&empty_w[i], GPS * 4);
        }
        for (int i = 0; i < XT; ++i) {
            mbar_init(&full_x[i], 1);
            mbar_init(&empty_x[i], 1);
            mbar_init(&x_tma[i], 1);
        }
        for (int i = 0; i < NA; ++i) {
            mbar_init(&a_full[i], 4);
            mbar_init(&a_free[i], 1);
        }
        mbar_init(d_full, 1);
        mbar_init(d_free, 4);
        mbar_init(red_bar, p.split > 1 ? (uint32_t)(p.split - 1) * 128u : 1u);
        mbar_fence_init();
    }
    if (warp == kTmaWarp) tmem_alloc(tmem_slot, (uint32_t)p.tmem_cols);
    for (uint32_t o = threadIdx.x * 16u; o < (uint32_t)XT * p.xt_bytes; o += kThreads * 16u)
        sts128(xt0 + o, make_uint4(0u, 0u, 0u, 0u));
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (p.split > 1) cluster_sync_all();      // every CTA's barriers exist before a neighbour arrives on one
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    pdl_launch_dependents();

    // ================================ TMA producer ================================================
    if (warp == kTmaWarp) {
        if (lane == 0) {
            bool ok = true;
            int slot = 0;
            uint32_t par = 0;
            const uint32_t tx = MATS * (kWTile + kMetaTile * (p.has_z ? 2 : 1));
            for (int ti = 0; ti < my_tiles; ++ti) {
                const int n0 = (cluster_id + ti * n_clusters) * kRows;
                for (int s = st_lo; s < st_hi; ++s) {
                    wait_bar(&empty_w[slot], par ^ 1u, EV_GEMV_EMPTY_WAIT, ok);
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
                    if (++slot == NS) { slot = 0; par ^= 1u; }
                }
            }
        }
    }
    // ================================ MMA issuer ==================================================
    else if (warp == kMmaWarp) {
        {
            bool ok = true;
            const uint32_t idesc = (1u << 4) | ((uint32_t)(ncols >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
            // K-major, 128-byte swizzle, 8-row groups 1024 bytes apart, descriptor version 1
            const uint64_t desc_hi = ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61) | (1ull << 16);
            int xslot = 0, a_slot = 0;
            uint32_t xpar = 0, a_par = 0;
            const uint32_t a_base = tmem + (uint32_t)p.a_col0;
            const uint32_t atom16 = (uint32_t)(ncols * 128) >> 4;      // distance of two 64-k atoms of the tile, in 16-byte units
            for (int ti = 0; ti < my_tiles; ++ti) {
                if (ti > 0) wait_bar(d_free, (uint32_t)(ti - 1) & 1u, EV_GEMV_EMPTY_WAIT, ok);
                tc_fence_after();
                for (int sl = 0; sl < n_st; ++sl) {
                    wait_bar(&full_x[xslot], xpar, EV_GEMV_FULL_WAIT, ok);
                    const uint32_t xb = xt0 + (uint32_t)xslot * p.xt_bytes;
                    // descriptor of the first K step of the stage's operand tile; the later steps are constant offsets
                    const uint64_t desc0 = desc_hi | (uint64_t)((xb & 0x3FFFFu) >> 4);
#pragma unroll
                    for (int u = 0; u < APS; ++u) {
                        const int c = u / MATS, m = u % MATS;
                        wait_bar(&a_full[a_slot], a_par, EV_GEMV_FULL_WAIT, ok);
                        tc_fence_after();
                        const uint32_t a_t = a_base + (uint32_t)a_slot * kChunkCols;
                        const uint32_t d_t = tmem + (uint32_t)(m * ncols);
                        const uint64_t desc_c = desc0 + (uint64_t)(c * 2) * atom16;
                        tc_mma_ts(d_t, a_t, desc_c, idesc, (sl == 0 && c == 0) ? 0u : 1u);
#pragma unroll
                        for (int i = 1; i < kChunkK / 16; ++i)
                            tc_mma_ts(d_t, a_t + i * 8, desc_c + (uint64_t)((i >> 2) * atom16 + (i & 3) * 2), idesc, 1u);
                        tc_commit(&a_free[a_slot]);
                        if (++a_slot == NA) { a_slot = 0; a_par ^= 1u; }
                    }
                    tc_commit(&empty_x[xslot]);
                    if (++xslot == XT) { xslot = 0; xpar ^= 1u; }
                }
                tc_commit(d_full);
            }
        }
    }
    // ================================ activation warps ============================================
    else if (warp >= kXWarp0) {
        pdl_wait();
        const int xw = warp - kXWarp0;
        constexpr int PPR = KS / 8;                            // 16-byte pieces per batch row and stage
        const int n_pieces = B * PPR;
        const int total_st = my_tiles * n_st;
        const uint32_t res0 = base + p.off_res;
        // Every activation warp owns the stages q = xw, xw + kXWarps, ... (the fixed cost of finishing a stage - waits,
        // proxy fence, arrival - is then paid once per kXWarps stages).  One TMA copy per 64 k puts the stage's rows
        // straight into the operand tile (the 128-byte swizzle of the copy IS the operand layout); the warp then
        // rewrites the pieces in place where needed (order of the codes for q4, rmsnorm) and hands the tile to the
        // MMA warp.  With more tiles than activation warps the copies of the warp's next stage are in flight while
        // it finishes the current one.
        const int my_total = total_st > xw ? (total_st - xw + kXWarps - 1) / kXWarps : 0;
        const int ahead = (XT > kXWarps && my_total > 1) ? 1 : 0;
        bool ok = true;
        auto tile_addr = [&](uint32_t tile, int idx) -> uint32_t {
            const int b = idx / PPR;
            const int pc = idx - b * PPR;
            return tile + (uint32_t)(pc >> 3) * (uint32_t)(ncols * 128) + (uint32_t)(b >> 3) * 1024u + (uint32_t)(b & 7) * 128u +
                   (uint32_t)(((pc & 7) ^ (b & 7)) << 4);
        };
        const uint32_t x_tx = (uint32_t)B * KS * 2 * (p.res_in != nullptr ? 2u : 1u);
        auto issue = [&](int q) {
            const int slot = q % XT;
            // the tile may still be read by the MMAs of the stage that used the slot before
            wait_bar(&empty_x[slot], (((uint32_t)q / (uint32_t)XT) & 1u) ^ 1u, EV_GEMV_EMPTY_WAIT, ok);
            if (lane == 0) {
                uint8_t* tile = sbase + p.off_xt + (size_t)slot * p.xt_bytes;
                uint8_t* res = sbase + p.off_res + (size_t)slot * p.res_bytes;
                const int k0 = (st_lo + q % n_st) * KS;
                mbar_arrive_expect_tx(&x_tma[slot], x_tx);
#pragma unroll
                for (int at = 0; at < KS / 64; ++at) {
                    tma_load_2d(tile + (size_t)at * ncols * 128, &p.xmap, (k0 + at * 64) * 2, 0, &x_tma[slot]);      // byte coordinates
                    if (p.res_in != nullptr) tma_load_2d(res + (size_t)at * B * 128, &p.rmap, (k0 + at * 64) * 2, 0, &x_tma[slot]);
                }
            }
            __syncwarp();
        };
        if (my_total > 0) issue(xw);
        // rmsnorm prologue: one warp per batch row; with more rows than activation warps the dequantise warps take
        // their share (they cannot get far before the first operand tile exists anyway)
        if (p.norm_w != nullptr) {
            const bool shared = B > kXWarps;
            const int nw = shared ? kXWarps + DW : kXWarps;
            for (int b = xw; b < B; b += nw) {
                const float inv = row_inv_rms(p, b, lane);
                if (lane == 0) inv_rms[b] = inv;
            }
            named_bar_sync(1, nw * 32);
        }
        const bool writes_side = cluster_id == 0;              // the cluster of tile 0 covers the whole K range
        for (int j = 0, q = xw; j < my_total; ++j, q += kXWarps) {
            if (ahead) {
                if (j + 1 < my_total) issue(q + kXWarps);
            } else if (j > 0) {
                issue(q);                                       // no spare tile: copy, then finish, one stage at a time
            }
            const int slot = q % XT;
            wait_bar(&x_tma[slot], ((uint32_t)q / (uint32_t)XT) & 1u, EV_GEMV_FULL_WAIT, ok);
            const uint32_t tile = xt0 + (uint32_t)slot * p.xt_bytes;
            const uint32_t res = res0 + (uint32_t)slot * p.res_bytes;
            const int k0 = (st_lo + q % n_st) * KS;
            if (p.norm_w == nullptr) {
                if (BITS == 4) {
                    // q4: piece (row i, lane) of the tile; the order in which the dequantise warps emit the 8 codes of a
                    // 32-bit word is (0,4) (1,5) (2,6) (3,7).  Four pieces in flight per lane.
                    const uint32_t lane_base = tile + (uint32_t)(lane >> 3) * (uint32_t)(ncols * 128) + (uint32_t)((lane & 7) << 4);
                    for (int i0 = 0; i0 < B; i0 += 4) {
                        uint4 u[4];
                        uint32_t addr[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int i = i0 + e < B ? i0 + e : i0;
                            addr[e] = (lane_base ^ (uint32_t)((i & 7) << 4)) + (uint32_t)(i >> 3) * 1024u + (uint32_t)(i & 7) * 128u;
                            u[e] = lds128(addr[e]);
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            u[e] = make_uint4(prmt(u[e].x, u[e].z, 0x5410), prmt(u[e].x, u[e].z, 0x7632), prmt(u[e].y, u[e].w, 0x5410),
                                              prmt(u[e].y, u[e].w, 0x7632));
                            if (i0 + e < B) sts128(addr[e], u[e]);
                        }
                    }
                }
            } else {
                // rows z = cast(x + residual), then cast(z * inv_rms * w): a lane meets the same 8 k of every row it
                // handles (32 % PPR == 0), so the norm weights are fetched once per stage
                const int pc = lane % PPR;
                const int k = k0 + pc * 8;
                float w8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) w8[i] = load_as_f32(p.norm_w, p.norm_w_dtype, k + i);
                const bool side = q < n_st && writes_side;          // first tile of the cluster that owns tile 0
                for (int idx = lane; idx < n_pieces; idx += 32) {
                    const int b = idx / PPR;
                    const uint32_t addr = tile_addr(tile, idx);
                    uint4 u = lds128(addr);
                    const __half2* hx = reinterpret_cast<const __half2*>(&u);
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) { v[2 * i] = __low2float(hx[i]); v[2 * i + 1] = __high2float(hx[i]); }
                    if (p.res_in != nullptr) {
                        const uint4 ur = lds128(res + (uint32_t)(pc >> 3) * (uint32_t)(B * 128) + (uint32_t)b * 128u + (uint32_t)((pc & 7) << 4));
                        const __half2* hr = reinterpret_cast<const __half2*>(&ur);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            v[2 * i] = __half2float(__float2half_rn(v[2 * i] + __low2float(hr[i])));
                            v[2 * i + 1] = __half2float(__float2half_rn(v[2 * i + 1] + __high2float(hr[i])));
                        }
                    }
                    if (side && p.z_out != nullptr) {
                        __half2 zo[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) zo[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                        *reinterpret_cast<uint4*>(p.z_out + (size_t)b * p.K + k) = *reinterpret_cast<const uint4*>(zo);
                    }
                    const float inv = inv_rms[b];
                    __half2 no[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) no[i] = __floats2half2_rn(v[2 * i] * inv * w8[2 * i], v[2 * i + 1] * inv * w8[2 * i + 1]);
                    u = *reinterpret_cast<const uint4*>(no);
                    if (side && p.normed_out != nullptr) *reinterpret_cast<uint4*>(p.normed_out + (size_t)b * p.K + k) = u;
                    if (BITS == 4)
                        u = make_uint4(prmt(u.x, u.z, 0x5410), prmt(u.x, u.z, 0x7632), prmt(u.y, u.w, 0x5410), prmt(u.y, u.w, 0x7632));
                    sts128(addr, u);
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_x[slot]);
        }
    }
    // ================================ dequantise warps (+ epilogue on warps 0-3) ===================
    else {
        const int grp = warp >> 2;                             // chunks a with a % NG == grp
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                     // weight row inside the tile = lane of tensor memory
        const uint32_t sw = (uint32_t)(r & 7);
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        bool ok = true;
        bool waited_pdl = false;
        if (p.norm_w != nullptr && B > kXWarps) {
            pdl_wait();
            waited_pdl = true;
            for (int b = kXWarps + warp; b < B; b += kXWarps + DW) {
                const float inv = row_inv_rms(p, b, lane);
                if (lane == 0) inv_rms[b] = inv;
            }
            named_bar_sync(1, (kXWarps + DW) * 32);
        }
        uint32_t a0 = 0;                     // index of the first chunk of A of the current stage (counted over the kernel)
        int slot = 0, t = grp % NA;          // ring positions of the stage and of this group's next chunk of A
        uint32_t par = 0, a_par = (uint32_t)(grp / NA) & 1u;
        for (int ti = 0; ti < my_tiles; ++ti) {
            const int n0 = (cluster_id + ti * n_clusters) * kRows;
            for (int s = st_lo; s < st_hi; ++s, a0 += APS) {
                // this group's chunks of the stage: u with (a0 + u) % NG == grp
                const int u0 = (int)((grp - (int)(a0 & (NG - 1)) + NG) & (NG - 1));
                if (u0 < APS) {
                    wait_bar(&full_w[slot], par, EV_GEMV_FULL_WAIT, ok);
                    const uint32_t st = stage0 + slot * p.stage_bytes;
#pragma unroll 1
                    for (int u = u0; u < APS; u += NG) {
                        const int c = u / MATS, m = u % MATS;
                        wait_bar(&a_free[t], a_par ^ 1u, EV_GEMV_EMPTY_WAIT, ok);
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
                        t += NG;
                        while (t >= NA) { t -= NA; a_par ^= 1u; }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty_w[slot]);
                }
                if (++slot == NS) { slot = 0; par ^= 1u; }
            }
            // ---- epilogue of the tile (split == 1; with a split K range it follows the cluster exchange below) ----
            if (warp < 4 && p.split == 1) {
                if (!waited_pdl) { pdl_wait(); waited_pdl = true; }
                const int n = n0 + r;
                float res[32];
                ts_load_residual<MATS>(p, n, res);
                wait_bar(d_full, (uint32_t)ti & 1u, EV_GEMV_FULL_WAIT, ok);
                tc_fence_after();
                {
                    float acc[MATS][16];
#pragma unroll
                    for (int m = 0; m < MATS; ++m) tc_ld16(lane_addr + (uint32_t)(m * ncols), acc[m]);
                    if (n < p.N) ts_store_cols<MATS, 0>(p, acc, n, res);
                }
                if (ncols > 16 && B > 16) {
                    float acc[MATS][16];
#pragma unroll
                    for (int m = 0; m < MATS; ++m) tc_ld16(lane_addr + (uint32_t)(m * ncols + 16), acc[m]);
                    if (n < p.N) ts_store_cols<MATS, 16>(p, acc, n, res);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(d_free);
            }
        }
    }

    // ---- split K range: the cluster's partial accumulators are summed in rank order by its first CTA (one tile
    //      per cluster).  Small batches send only their real columns into a dedicated buffer and signal a barrier
    //      of the first CTA; otherwise the first CTA's weight ring is reused between two cluster-wide barriers. ----
    if (p.split > 1) {
        __syncwarp();
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        const bool fast = p.off_red != 0;
        const int rcols = fast ? B : ncols;                  // columns per matrix that travel
        const uint32_t red_base = fast ? base + p.off_red : stage0;
        const bool epi = warp < 4 && my_tiles > 0;
        bool ok = true;
        if (epi) {
            wait_bar(d_full, 0u, EV_GEMV_FULL_WAIT, ok);
            tc_fence_after();
        }
        if (!fast) cluster_sync_all();      // every CTA of the cluster is done with its ring: the first CTA's ring is free
        if (epi && rank != 0) {
            for (int m = 0; m < MATS; ++m)
                for (int c0 = 0; c0 < rcols; c0 += 16) {
                    float acc[16];
                    tc_ld16(lane_addr + (uint32_t)(m * ncols + c0), acc);
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < rcols)
                            st_cluster_f32(red_base + (uint32_t)(((((int)rank - 1) * MATS + m) * rcols + c0 + j) * kRows + r) * 4u, 0u, acc[j]);
                }
            if (fast) arrive_remote(smem_u32(red_bar), 0u);
        }
        if (!fast) cluster_sync_all();      // the partial sums are in the first CTA's shared memory
        if (epi && rank == 0) {
            pdl_wait();
            const int n = cluster_id * kRows + r;
            float res[32];
            ts_load_residual<MATS>(p, n, res);
            if (fast) wait_bar_cluster(red_bar, 0u, ok ? kTsWaitLimit : 64u);
            const float* red = reinterpret_cast<const float*>(sbase + (red_base - base));
#pragma unroll
            for (int c0 = 0; c0 < 32; c0 += 16) {
                if (c0 >= rcols) break;
                float acc[MATS][16];
#pragma unroll
                for (int m = 0; m < MATS; ++m) {
                    tc_ld16(lane_addr + (uint32_t)(m * ncols + c0), acc[m]);
                    for (int q = 1; q < p.split; ++q)
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < rcols) acc[m][j] += red[((((q - 1) * MATS + m) * rcols + c0 + j) * kRows + r)];
                }
                if (n < p.N) {
                    if (c0 == 0) ts_store_cols<MATS, 0>(p, acc, n, res);
                    else ts_store_cols<MATS, 16>(p, acc, n, res);
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

template <int BITS, int LOGG, int MATS, bool WHOLE>
int launch_ts(TsParams& p, cudaStream_t stream) {
    constexpr int KS = kRowBytes * 8 / BITS;
    const int sms = sm_count();
    p.n_stage_total = p.K / KS;
    p.tiles = (p.N + kRows - 1) / kRows;
    p.off_meta = MATS * kWTile;
    p.stage_bytes = MATS * (kWTile + 2 * kMetaTile);
    p.xt_bytes = (uint32_t)p.ncols * KS * 2;
    p.res_bytes = p.res_in != nullptr ? (uint32_t)p.B * KS * 2 : 0u;
    // compact shape: a CTA stays below half of an SM's shared memory, registers and tensor memory
    const uint32_t cap = (uint32_t)max_smem_optin();
    uint32_t budget = WHOLE ? cap : std::min<uint32_t>(cap, 112u * 1024u);
    const int forced = tuning_get("ts.smem_kb");
    if (forced > 0) budget = std::min<uint32_t>(cap, (uint32_t)forced * 1024u);
    // tensor memory: accumulators below, ring of A chunks above
    const int dcols = MATS * p.ncols;
    p.a_col0 = std::max(32, (dcols + 31) / 32 * 32);
    p.tmem_cols = WHOLE ? 512 : 256;
    p.a_slots = std::min(kMaxASlots, (p.tmem_cols - p.a_col0) / kChunkCols);
    if (p.a_slots < 2) return B200Q_ERR_UNSUPPORTED;
    // K split over a cluster when the tiles do not fill the SMs.  The split (and with it the order in which a row's
    // partial sums are added) must not depend on how many rows THIS launch holds: a tensor-parallel shard of the rows
    // has to reproduce the unsharded result bit for bit, so the tile count of the unsharded matrix decides
    // ("ts.tp_world" = number of equal row shards), and the cap below uses no shape-dependent quantity.
    const int tiles_full = p.tiles * std::max(1, tuning_get("ts.tp_world"));
    int split = 1;
    if (tiles_full < sms) split = std::min(8, sms / tiles_full);
    split = std::max(1, std::min(split, p.n_stage_total / 2));
    // the partial sums of the other CTAs of a cluster (real batch columns only) must fit 48 KB of the first CTA's
    // shared memory; like the split itself the bound depends on the batch alone, not on the shape of this launch
    constexpr uint32_t kRedCap = 48u * 1024u;
    const uint32_t part_bytes = (uint32_t)MATS * p.B * kRows * 4;
    if ((uint32_t)(split - 1) * part_bytes > kRedCap) split = std::max(1, std::min(split, 1 + (int)(kRedCap / part_bytes)));
    const int fs = tuning_get("ts.split");
    if (fs > 0) split = std::max(1, std::min({fs, 8, p.n_stage_total}));
    // they arrive in a dedicated buffer signalled by a barrier (whole-SM shape: up to the 48 KB, compact shape: 8 KB),
    // else in the first CTA's weight ring between two cluster-wide barriers; both add them in rank order
    const uint32_t red_bytes = (uint32_t)(split - 1) * part_bytes;
    const bool fast_red = split > 1 && red_bytes <= (WHOLE ? kRedCap : 8192u) && !tuning_get("ts.slow_reduce");
    const uint32_t red_alloc = fast_red ? (red_bytes + 1023u) / 1024u * 1024u : 0u;
    // rings: operand tiles (at least as many as activation warps: a warp must never meet a tile slot two uses ahead of
    // the MMAs; one more lets it keep the copies of its next stage in flight), then as many weight stages as fit
    constexpr int XW = ts_xwarps(WHOLE);
    const uint32_t per_tile = p.xt_bytes + p.res_bytes;
    const uint32_t base_fixed = 2048u + red_alloc;
    int xt = XW + 2;
    while (xt > XW && base_fixed + (uint32_t)xt * per_tile + 3 * p.stage_bytes > budget) --xt;
    p.x_tiles = std::min(xt, kMaxXTiles);
    const uint32_t fixed = base_fixed + (uint32_t)p.x_tiles * per_tile;
    if (fixed + 2 * p.stage_bytes > budget) return B200Q_ERR_UNSUPPORTED;
    int stages = (int)((budget - fixed) / p.stage_bytes);
    const int want = tuning_get("ts.stages");
    if (want > 0) stages = std::min(stages, want);
    stages = std::min(stages, kMaxStages);
    if (stages < 2) return B200Q_ERR_UNSUPPORTED;
    p.stages = stages;
    if (!fast_red && split > 1 && (uint64_t)(split - 1) * dcols * kRows * 4 > (uint64_t)stages * p.stage_bytes)
        return B200Q_ERR_UNSUPPORTED;      // only with a forced split
    p.split = split;
    p.off_xt = 1024u + (uint32_t)stages * p.stage_bytes;
    p.off_res = p.off_xt + (uint32_t)p.x_tiles * p.xt_bytes;
    p.off_red = (fast_red && split > 1) ? p.off_res + (uint32_t)p.x_tiles * p.res_bytes : 0u;
    const int clusters = split > 1 ? p.tiles : std::min(p.tiles, sms);
    const uint32_t smem = 1024u + p.off_res + (uint32_t)p.x_tiles * p.res_bytes + red_alloc;

    auto kernel = qgemm_ts_kernel<BITS, LOGG, MATS, WHOLE>;
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
    cfg.blockDim = dim3(ts_threads(WHOLE));
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

// The whole-SM shape for matrices large enough that the depth of the rings matters more than overlapping the head
// of the next kernel (measured: 16 MB of codes and up), and whenever the compact shape does not fit;
// "ts.big" = 1 / -1 forces / prefers the other.
template <int BITS, int LOGG, int MATS>
int launch_ts_shape(TsParams& p, int64_t weight_bytes, cudaStream_t stream) {
    const int mode = tuning_get("ts.big");
    // (the size of the UNSHARDED matrix decides, so that a tensor-parallel shard runs the shape, and with it the K
    // split, of the unsharded launch)
    const int64_t full_bytes = weight_bytes * std::max(1, tuning_get("ts.tp_world"));
    const bool big = mode > 0 || (mode == 0 && full_bytes >= (int64_t)16 << 20);
    if (!big) {
        const int rc = launch_ts<BITS, LOGG, MATS, false>(p, stream);
        if (rc != B200Q_ERR_UNSUPPORTED) return rc;
    }
    return launch_ts<BITS, LOGG, MATS, true>(p, stream);
}

template <int BITS>
int dispatch_ts(TsParams& p, int G, bool gate_up, int64_t weight_bytes, cudaStream_t stream) {
    if (gate_up) {
        if (G == 32) return launch_ts_shape<BITS, 5, 2>(p, weight_bytes, stream);
        if (G == 64) return launch_ts_shape<BITS, 6, 2>(p, weight_bytes, stream);
        return launch_ts_shape<BITS, 7, 2>(p, weight_bytes, stream);
    }
    if (G == 32) return launch_ts_shape<BITS, 5, 1>(p, weight_bytes, stream);
    if (G == 64) return launch_ts_shape<BITS, 6, 1>(p, weight_bytes, stream);
    return launch_ts_shape<BITS, 7, 1>(p, weight_bytes, stream);
}

}  // namespace

// Returns B200Q_ERR_UNSUPPORTED when the problem is outside this kernel (the caller then uses the other kernels).
int qgemm_ts(int bits, const GemvParams& g, bool gate_up, cudaStream_t stream) {
    if (g.act_dtype != B200Q_F16 || g.scale_dtype != B200Q_F16) return B200Q_ERR_UNSUPPORTED;
    if (g.G != 32 && g.G != 64 && g.G != 128) return B200Q_ERR_UNSUPPORTED;
    const int KS = kRowBytes * 8 / bits;
    if (g.K % KS != 0 || g.K % g.G != 0 || g.Gn % 8 != 0 || g.row_bytes % 16 != 0) return B200Q_ERR_UNSUPPORTED;
    if (g.B > 32 || g.tp_in.world > 0 || g.tp_out.world > 0) return B200Q_ERR_UNSUPPORTED;    // larger batches: 32 rows per launch
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
    if (!tensor_map_2d(g.x, (uint64_t)g.K * 2, (uint64_t)g.B, 128, (uint32_t)g.B, true, &p.xmap)) return B200Q_ERR_UNSUPPORTED;
    if (g.res_in != nullptr && !tensor_map_2d(g.res_in, (uint64_t)g.K * 2, (uint64_t)g.B, 128, (uint32_t)g.B, false, &p.rmap))
        return B200Q_ERR_UNSUPPORTED;
    p.x = (const __half*)g.x; p.res_in = (const __half*)g.res_in; p.norm_w = g.norm_w; p.norm_w_dtype = g.norm_w_dtype;
    p.z_out = (__half*)g.z_out; p.normed_out = (__half*)g.normed_out; p.residual = (const __half*)g.residual;
    p.y = (__half*)g.y; p.gate_out = (__half*)g.gate_out; p.up_out = (__half*)g.up_out; p.act_out = (__half*)g.act_out;
    p.eps = g.eps; p.B = g.B; p.N = g.N; p.K = g.K; p.has_z = g.z[0] != nullptr ? 1 : 0;
    p.ncols = (g.B + 15) / 16 * 16;
    const int64_t weight_bytes = (int64_t)mats * g.N * g.row_bytes;
    return bits == 4 ? dispatch_ts<4>(p, g.G, gate_up, weight_bytes, stream) : dispatch_ts<8>(p, g.G, gate_up, weight_bytes, stream);
}


}  // namespace b200q
