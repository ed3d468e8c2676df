// Oracle (test infrastructure): runs the reference's own Metal kernel bodies on the CPU.
//
// The hot-path kernels of manishklach/mlx-metal-kernels are Metal Shading Language *bodies*
// (no signature; MLX generates it).  The one-thread-per-output bodies are plain C apart from
// `thread_position_in_grid`, `ELEM_TYPE` and a few math names, so they compile as C++ when
// they are #included inside a lambda that is called once per thread id.  Nothing is copied:
// the build (oracle/Makefile) passes -I<reference>/kernels and the preprocessor reads the
// .metal files where they lie.  Output goes to oracle/_ref/libmetalref.so.
//
// Used only by tests to pin oracle/*.py against code the reference ships.
#include <cmath>
#include <cstdint>
#include <algorithm>

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
