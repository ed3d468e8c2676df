// Oracle (test infrastructure): runs the reference's own Metal kernel bodies on the CPU.
//
// The hot-path kernels of manishklach/mlx-metal-kernels are Metal Shading Language *bodies*
// (no signature; MLX generates it).  The one-thread-per-output bodies are plain C apart from
// `thread_position_in_grid`, `ELEM_TYPE` and a few math names, so they compile as C++ when
// they are #included inside a lambda that is called once per thread id.  Nothing is copied:
// the build (oracle/Makefile) passes -I<reference>/kernels and the preprocessor reads the
// .metal files where they lie.  Output goes to oracle/_ref/libmetalref.so.
//
// The bodies that cooperate inside a threadgroup (threadgroup arrays, threadgroup_barrier, simd_sum) run on a small
// emulator further down: one std::thread per GPU thread of a group, a std::barrier for the group and one per
// simdgroup; groups run one after the other.
//
// Used only by tests to pin oracle/*.py against code the reference ships.
#include <cmath>
#include <cstdint>
#include <algorithm>
#include <barrier>
#include <memory>
#include <thread>
#include <vector>

using std::exp;
using std::isfinite;
using std::max;
using std::min;

typedef unsigned int uint;
typedef unsigned char uchar;
typedef _Float16 half;
typedef __bf16 bfloat;

#define MAX_HEAD_DIM 128

struct GridPos { uint x; };

// GRID_BEGIN/GRID_END run the enclosed body once per thread id in [0, grid); a `return`
// inside a body leaves the lambda only, like an early exit of one GPU thread.
#define GRID_BEGIN(grid)                                                  \
    for (long long tid_ = 0; tid_ < (long long)(grid); ++tid_) {          \
        const GridPos thread_position_in_grid{(uint)tid_};                \
        [&]() {
#define GRID_END                                                          \
        }();                                                              \
    }

// ---- kernels/dequant_q4.metal, kernels/dequant_q8.metal ---------------------------------
#define ELEM_TYPE half
extern "C" void ref_dequant_q4_f16(const uint8_t* packed, const float* scales, const float* zeros,
                                   const int* meta, half* out, long long grid) {
    GRID_BEGIN(grid)
#include "dequant_q4.metal"
    GRID_END
}
extern "C" void ref_dequant_q8_f16(const uint8_t* q, const float* scales, const float* zeros,
                                   const int* meta, half* out, long long grid) {
    GRID_BEGIN(grid)
#include "dequant_q8.metal"
    GRID_END
}
// ---- kernels/q4_matvec_decode.metal, kernels/q8_matvec_decode.metal ------------------------
extern "C" void ref_q4_matvec_f16(const half* x, const uint8_t* packed_w, const float* scales,
                                  const float* zeros, const int* meta, half* y, long long grid) {
    GRID_BEGIN(grid)
#include "q4_matvec_decode.metal"
    GRID_END
}
extern "C" void ref_q8_matvec_f16(const half* x, const uint8_t* q_w, const float* scales,
                                  const float* zeros, const int* meta, half* y, long long grid) {
    GRID_BEGIN(grid)
#include "q8_matvec_decode.metal"
    GRID_END
}
// ---- kernels/q{4,8}_paged_gqa_decode_attention.metal ---------------------------------------
extern "C" void ref_q4_paged_attn_f16(const half* q, const uint8_t* K_pages_q, const uint8_t* V_pages_q,
                                      const float* K_scales, const float* V_scales,
                                      const int* block_table, const int* lengths, const int* meta,
                                      const float* scale, half* out, long long grid) {
    GRID_BEGIN(grid)
#include "q4_paged_gqa_decode_attention.metal"
    GRID_END
}
extern "C" void ref_q8_paged_attn_f16(const half* q, const uint8_t* K_pages_q, const uint8_t* V_pages_q,
                                      const float* K_scales, const float* V_scales,
                                      const int* block_table, const int* lengths, const int* meta,
                                      const float* scale, half* out, long long grid) {
    GRID_BEGIN(grid)
#include "q8_paged_gqa_decode_attention.metal"
    GRID_END
}
// ---- kernels/q{4,8}_gqa_decode_attention.metal (contiguous cache) ----------------------------
extern "C" void ref_q4_attn_f16(const half* q, const uint8_t* K_q, const uint8_t* V_q, const float* K_scales,
                                const float* V_scales, const int* lengths, const int* meta, const float* scale,
                                half* out, long long grid) {
    GRID_BEGIN(grid)
#include "q4_gqa_decode_attention.metal"
    GRID_END
}
extern "C" void ref_q8_attn_f16(const half* q, const uint8_t* K_q, const uint8_t* V_q, const float* K_scales,
                                const float* V_scales, const int* lengths, const int* meta, const float* scale,
                                half* out, long long grid) {
    GRID_BEGIN(grid)
#include "q8_gqa_decode_attention.metal"
    GRID_END
}
// ---- kernels/fused_swiglu.metal ------------------------------------------------------------
extern "C" void ref_fused_swiglu_f16(const half* gate, const half* up, const int* meta, half* out,
                                     long long grid) {
    GRID_BEGIN(grid)
#include "fused_swiglu.metal"
    GRID_END
}
#undef ELEM_TYPE

#define ELEM_TYPE bfloat
extern "C" void ref_dequant_q4_bf16(const uint8_t* packed, const float* scales, const float* zeros,
                                    const int* meta, bfloat* out, long long grid) {
    GRID_BEGIN(grid)
#include "dequant_q4.metal"
    GRID_END
}
extern "C" void ref_dequant_q8_bf16(const uint8_t* q, const float* scales, const float* zeros,
                                    const int* meta, bfloat* out, long long grid) {
    GRID_BEGIN(grid)
#include "dequant_q8.metal"
    GRID_END
}
extern "C" void ref_q4_matvec_bf16(const bfloat* x, const uint8_t* packed_w, const float* scales,
                                   const float* zeros, const int* meta, bfloat* y, long long grid) {
    GRID_BEGIN(grid)
#include "q4_matvec_decode.metal"
    GRID_END
}
#undef ELEM_TYPE

// ---- kernels/block_table_lookup.metal (integer, no ELEM_TYPE) ------------------------------
extern "C" void ref_block_table_lookup(const int* block_table, const int* positions, const int* meta,
                                       int* page_ids, int* offsets, long long grid) {
    GRID_BEGIN(grid)
#include "block_table_lookup.metal"
    GRID_END
}

// ---- kernels/residual_add.metal, kernels/swiglu.metal (one thread per element) -----------------
#define ELEM_TYPE half
extern "C" void ref_residual_add_f16(const half* x, const half* residual, const int* meta, half* y, long long grid) {
    GRID_BEGIN(grid)
#include "residual_add.metal"
    GRID_END
}
extern "C" void ref_swiglu_f16(const half* gate, const half* up, const int* meta, half* out, long long grid) {
    GRID_BEGIN(grid)
#include "swiglu.metal"
    GRID_END
}
#undef ELEM_TYPE

// ================================================================================================
// Threadgroup emulator
// ================================================================================================
namespace tg {
struct Group {
    uint size;
    std::barrier<> all;
    std::vector<std::unique_ptr<std::barrier<>>> simd;
    std::vector<float> lanes;            // [simdgroups][32] exchange buffer of simd_sum
    explicit Group(uint n) : size(n), all(n), lanes(((n + 31) / 32) * 32, 0.0f) {
        for (uint s = 0; s < (n + 31) / 32; ++s)
            simd.emplace_back(std::make_unique<std::barrier<>>(std::min(32u, n - 32 * s)));
    }
};
// Sum over the lanes of the caller's simdgroup in butterfly order (v += shuffle_xor(v, 16, 8, 4, 2, 1)); every lane
// gets the same bits.  Metal leaves the order of simd_sum to the implementation, so results pinned through it are
// compared with a rounding tolerance.
inline float simd_sum_impl(Group& g, uint tid, float v) {
    const uint sg = tid / 32, lane = tid % 32;
    const uint width = std::min(32u, g.size - 32 * sg);
    g.lanes[sg * 32 + lane] = v;
    g.simd[sg]->arrive_and_wait();
    float cur[32];
    for (uint i = 0; i < 32; ++i) cur[i] = i < width ? g.lanes[sg * 32 + i] : 0.0f;
    for (uint off = 16; off > 0; off >>= 1) {
        float nxt[32];
        for (uint i = 0; i < 32; ++i) nxt[i] = cur[i] + cur[i ^ off];
        for (uint i = 0; i < 32; ++i) cur[i] = nxt[i];
    }
    g.simd[sg]->arrive_and_wait();        // everyone has read the buffer before it is written again
    return cur[lane];
}
template <class Body> void run(uint groups, uint size, Body body) {
    for (uint gidx = 0; gidx < groups; ++gidx) {
        Group g(size);
        std::vector<std::thread> threads;
        threads.reserve(size);
        for (uint t = 0; t < size; ++t) threads.emplace_back([&, t]() { body(g, gidx, t); });
        for (auto& th : threads) th.join();
    }
}
}  // namespace tg

struct mem_flags { static constexpr int mem_threadgroup = 0; };
inline float rsqrt(float v) { return 1.0f / std::sqrt(v); }

// A body sees the Metal names it uses; `threadgroup` arrays become statics of the lambda (one instance, shared by the
// threads of the group; groups run one at a time and every body writes them before reading).
#define TG_BEGIN(n_groups_, n_threads_)                                                      \
    tg::run((uint)(n_groups_), (uint)(n_threads_), [&](tg::Group& tg_group_, uint tg_gidx_, uint tg_tid_) { \
        const GridPos thread_position_in_threadgroup{tg_tid_};                              \
        const GridPos threadgroup_position_in_grid{tg_gidx_};                               \
        const GridPos threads_per_threadgroup{tg_group_.size};                              \
        const GridPos thread_position_in_grid{tg_gidx_ * tg_group_.size + tg_tid_};         \
        const uint thread_index_in_simdgroup = tg_tid_ % 32;                                \
        const uint simdgroup_index_in_threadgroup = tg_tid_ / 32;                           \
        (void)thread_position_in_grid; (void)thread_index_in_simdgroup; (void)simdgroup_index_in_threadgroup;
#define TG_END });
#define threadgroup static
#define threadgroup_barrier(flags) tg_group_.all.arrive_and_wait()
#define simd_sum(v) tg::simd_sum_impl(tg_group_, tg_tid_, (v))
#define MATVEC_THREADS 128
#define MATVEC_TILED_THREADS 128

#define ELEM_TYPE half
// ---- kernels/rms_norm.metal, kernels/rmsnorm_residual.metal (one group of `threads` per row) ---
extern "C" void ref_rms_norm_f16(const half* x, const half* weight, const int* meta, const float* eps, half* y,
                                 long long groups, long long threads) {
    TG_BEGIN(groups, threads)
#include "rms_norm.metal"
    TG_END
}
extern "C" void ref_rmsnorm_residual_f16(const half* x, const half* residual, const half* weight, const int* meta,
                                         const float* eps, half* y, half* z, long long groups, long long threads) {
    TG_BEGIN(groups, threads)
#include "rmsnorm_residual.metal"
    TG_END
}
// ---- kernels/q{4,8}_matvec_decode_parallel.metal (one group per output), _tiled (four outputs per group) ----
extern "C" void ref_q4_matvec_parallel_f16(const half* x, const uint8_t* packed_w, const float* scales,
                                           const float* zeros, const int* meta, half* y, long long groups,
                                           long long threads) {
    TG_BEGIN(groups, threads)
#include "q4_matvec_decode_parallel.metal"
    TG_END
}
extern "C" void ref_q8_matvec_parallel_f16(const half* x, const uint8_t* q_w, const float* scales, const float* zeros,
                                           const int* meta, half* y, long long groups, long long threads) {
    TG_BEGIN(groups, threads)
#include "q8_matvec_decode_parallel.metal"
    TG_END
}
extern "C" void ref_q4_matvec_tiled_f16(const half* x, const uint8_t* packed_w, const float* scales, const float* zeros,
                                        const int* meta, half* y, long long groups, long long threads) {
    TG_BEGIN(groups, threads)
#include "q4_matvec_decode_tiled.metal"
    TG_END
}
extern "C" void ref_q8_matvec_tiled_f16(const half* x, const uint8_t* q_w, const float* scales, const float* zeros,
                                        const int* meta, half* y, long long groups, long long threads) {
    TG_BEGIN(groups, threads)
#include "q8_matvec_decode_tiled.metal"
    TG_END
}
// ---- kernels/q{4,8}_gate_up_matvec_tiled.metal --------------------------------------------------
extern "C" void ref_q4_gate_up_tiled_f16(const half* x, const uint8_t* gate_packed, const uint8_t* up_packed,
                                         const float* gate_scales, const float* up_scales, const float* gate_zeros,
                                         const float* up_zeros, const int* meta, half* gate, half* up, long long groups,
                                         long long threads) {
    TG_BEGIN(groups, threads)
#include "q4_gate_up_matvec_tiled.metal"
    TG_END
}
extern "C" void ref_q8_gate_up_tiled_f16(const half* x, const uint8_t* gate_q, const uint8_t* up_q,
                                         const float* gate_scales, const float* up_scales, const float* gate_zeros,
                                         const float* up_zeros, const int* meta, half* gate, half* up, long long groups,
                                         long long threads) {
    TG_BEGIN(groups, threads)
#include "q8_gate_up_matvec_tiled.metal"
    TG_END
}
#undef ELEM_TYPE
