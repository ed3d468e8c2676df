// C ABI of libb200q plus the small memory-bound kernels (dequant, SwiGLU, residual add,
// RMSNorm(+residual), block-table lookup).
#include "common.cuh"

#include <algorithm>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

namespace b200q {

// ------------------------------------------------------------------------------------------------
// host-side state: tuning table and cached device properties
// ------------------------------------------------------------------------------------------------
namespace {
std::mutex g_mu;
std::unordered_map<std::string, int> g_tuning;
struct DevProps { int sms = 0; int smem_optin = 0; };
DevProps g_props[64];

const DevProps& props() {
    int dev = 0;
    cudaGetDevice(&dev);
    DevProps& p = g_props[dev & 63];
    if (p.sms == 0) {
        std::lock_guard<std::mutex> lock(g_mu);
        if (p.sms == 0) {
            int sms = 0, smem = 0;
            cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            p.smem_optin = smem;
            p.sms = sms > 0 ? sms : 1;
        }
    }
    return p;
}
}  // namespace

namespace {
TpSlot g_tp_slots[16];
bool g_tp_valid[16] = {};
thread_local int g_tp_next_in = -1, g_tp_next_out = -1;
}  // namespace

const TpSlot* tp_slot(int slot) { return (slot >= 0 && slot < 16 && g_tp_valid[slot]) ? &g_tp_slots[slot] : nullptr; }
void tp_take(int* in_slot, int* out_slot) {
    *in_slot = g_tp_next_in;
    *out_slot = g_tp_next_out;
    g_tp_next_in = g_tp_next_out = -1;
}
void tp_discard() { g_tp_next_in = g_tp_next_out = -1; }

int tuning_get(const char* key) {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_tuning.find(key);
    return it == g_tuning.end() ? 0 : it->second;
}
int sm_count() { return props().sms; }
int max_smem_optin() { return props().smem_optin; }

// implemented in gemv.cu / paged_attn.cu
int gemv_read_status(int reset, cudaStream_t stream);
int attn_read_status(int reset, cudaStream_t stream);
int peer_read_status(int reset, cudaStream_t stream);
int stack_read_status(int reset, cudaStream_t stream);
int quantize_kv_impl(int bits, const void* values, uint8_t* codes, void* scales, int64_t rows, int D, int group_size,
                     int in_dtype, cudaStream_t stream);
int peer_allgather_impl(const void* local, void* const* peer_full, uint32_t* const* peer_flags, uint32_t* epoch,
                        int rank, int world, int rows, int64_t row_bytes_local, cudaStream_t stream);
int wait_expiry_selftest_impl(uint32_t limit, uint32_t* probes_out, cudaStream_t stream);
int qmatvec_impl(int bits, const void* x, const uint8_t* codes, const void* scales, const void* zeros,
                 const void* residual, void* y, int B, int64_t N, int64_t K, int group_size, int act_dtype,
                 int scale_dtype, const void* residual_in, const void* norm_weight, int norm_w_dtype, float eps,
                 void* z_out, void* normed_out, cudaStream_t stream);
int rope_kv_append_impl(const void* qkv, const float* cos_table, const float* sin_table, const int32_t* positions,
                        const int32_t* block_table, void* q_out, uint8_t* k_codes, uint8_t* v_codes, void* k_scales,
                        void* v_scales, int bits, int B, int Hq, int Hkv, int D, int page_size, int64_t num_pages,
                        int max_blocks, int group_size, int table_len, cudaStream_t stream);
int gate_up_impl(int bits, const void* x, const uint8_t* gate_codes, const uint8_t* up_codes, const void* gate_scales,
                 const void* up_scales, const void* gate_zeros, const void* up_zeros, void* gate_out, void* up_out,
                 void* act_out, const void* residual_in, const void* norm_weight, float eps, void* z_out,
                 void* normed_out, int rows, int64_t N, int64_t K, int group_size, int act_dtype, int scale_dtype,
                 int norm_w_dtype, cudaStream_t stream);
int rope_append_attention_impl(const void* qkv, const float* cos_table, const float* sin_table, const int32_t* positions,
                               int table_len, int bits, uint8_t* k_codes, uint8_t* v_codes, void* k_scales, void* v_scales,
                               const int32_t* block_table, const int32_t* lengths, void* out, void* q_scratch, void* workspace,
                               size_t workspace_bytes, int B, int Hq, int Hkv, int D, int page_size, int64_t num_pages,
                               int max_blocks, int group_size, float scale, cudaStream_t stream);
int paged_gqa_decode_block_sparse_impl(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                                       const void* k_scales, const void* v_scales, const int32_t* block_table,
                                       const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes,
                                       const uint8_t* block_mask, int n_qblocks, int n_kblocks, int block_size,
                                       int32_t* page_scratch, int B, int Hq, int Hkv, int D, int page_size,
                                       int64_t num_pages, int max_blocks, int group_size, float scale, int q_dtype,
                                       int scale_dtype, cudaStream_t stream);
size_t paged_fp16_workspace_bytes_impl(int B, int Hq, int Hkv, int max_blocks);
int paged_fp16_gqa_decode_impl(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_table,
                               const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes, int B, int Hq,
                               int Hkv, int D, int page_size, int64_t num_pages, int max_blocks, float scale, int dtype,
                               cudaStream_t stream);
size_t paged_gqa_workspace_bytes_impl(int B, int Hq, int Hkv, int D);
int attention_stage_launches_impl(int B, int Hkv, int with_append);
size_t paged_gqa_static_scratch_bytes_impl();
int paged_gqa_decode_static_impl(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                                 const void* k_scales, const void* v_scales, const int32_t* block_table,
                                 const int32_t* lengths, void* out, int B, int Hq, int Hkv, int D, int page_size,
                                 int64_t num_pages, int max_blocks, int group_size, float scale, int q_dtype,
                                 int scale_dtype, cudaStream_t stream);
int paged_gqa_decode_impl(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes, const void* k_scales,
                          const void* v_scales, const int32_t* block_table, const int32_t* lengths, void* out,
                          void* workspace, size_t workspace_bytes, int B, int Hq, int Hkv, int D, int page_size,
                          int64_t num_pages, int max_blocks, int group_size, float scale, int q_dtype,
                          int scale_dtype, int sink_tokens, int window_size, cudaStream_t stream);

// ------------------------------------------------------------------------------------------------
// dequant: out = cast(fp32(code - zero) * scale).  __fsub_rn / __fmul_rn keep the two roundings
// separate (no contraction), which is what makes the result bit-identical to the reference.
// One thread produces 8 consecutive outputs (a 16-byte store).
// ------------------------------------------------------------------------------------------------
namespace {

template <typename OUT>
__global__ void __launch_bounds__(256) dequant_kernel(int bits, const uint8_t* __restrict__ codes,
                                                      const void* __restrict__ scales, const void* __restrict__ zeros,
                                                      OUT* __restrict__ out, int64_t M, int64_t K, int G, int Gn,
                                                      int64_t row_bytes, int scale_dtype, bool vec_ok) {
    const int64_t k8 = (K + 7) / 8;
    const int64_t total = M * k8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / k8;
        const int64_t k0 = (i - m * k8) * 8;
        const uint8_t* row = codes + m * row_bytes;
        float v[8];
        uint32_t lo = 0, hi = 0;
        const bool full = k0 + 8 <= K;
        if (full && vec_ok) {
            if (bits == 4) {
                lo = *reinterpret_cast<const uint32_t*>(row + k0 / 2);
            } else {
                const uint2 u = *reinterpret_cast<const uint2*>(row + k0);
                lo = u.x;
                hi = u.y;
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t k = k0 + j;
            if (k >= K) { v[j] = 0.0f; continue; }
            uint32_t code;
            if (full && vec_ok) {
                code = bits == 4 ? (lo >> (4 * j)) & 0xF : ((j < 4 ? lo >> (8 * j) : hi >> (8 * (j - 4))) & 0xFF);
            } else if (bits == 4) {
                const uint8_t byte = row[k >> 1];
                code = (k & 1) ? (byte >> 4) : (byte & 0xF);
            } else {
                code = row[k];
            }
            const int64_t gi = m * Gn + k / G;
            const float s = load_as_f32(scales, scale_dtype, gi);
            const float q = (float)code;
            v[j] = zeros != nullptr ? __fmul_rn(__fsub_rn(q, load_as_f32(zeros, scale_dtype, gi)), s) : __fmul_rn(q, s);
        }
        OUT* dst = out + m * K + k0;
        if (full && vec_ok) {
            OUT tmp[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) tmp[j] = from_f32<OUT>(v[j]);
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(tmp);
        } else {
            for (int j = 0; j < 8 && k0 + j < K; ++j) dst[j] = from_f32<OUT>(v[j]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                                                     T* __restrict__ out, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float g = to_f32(gate[i]);
        const float u = to_f32(up[i]);
        out[i] = from_f32<T>((g / (1.0f + expf(-g))) * u);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) residual_add_kernel(const T* __restrict__ x, const T* __restrict__ r,
                                                           T* __restrict__ out, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(to_f32(x[i]) + to_f32(r[i]));
}

// one CTA per row
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_residual_kernel(const T* __restrict__ x, const T* __restrict__ res,
                                                               const void* __restrict__ w, T* __restrict__ y,
                                                               T* __restrict__ z_out, int64_t D, float eps, int w_dtype) {
    __shared__ float warp_part[8];
    __shared__ float inv_rms;
    const int64_t row = blockIdx.x;
    const T* xr = x + row * D;
    const T* rr = res ? res + row * D : nullptr;
    float ss = 0.0f;
    for (int64_t i = threadIdx.x; i < D; i += blockDim.x) {
        float z = to_f32(xr[i]);
        if (rr) z = to_f32(from_f32<T>(z + to_f32(rr[i])));
        ss += z * z;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += warp_part[i];
        inv_rms = rsqrtf(t / (float)D + eps);
    }
    __syncthreads();
    const float inv = inv_rms;
    for (int64_t i = threadIdx.x; i < D; i += blockDim.x) {
        float z = to_f32(xr[i]);
        if (rr) z = to_f32(from_f32<T>(z + to_f32(rr[i])));
        if (z_out) z_out[row * D + i] = from_f32<T>(z);
        y[row * D + i] = from_f32<T>(z * inv * load_as_f32(w, w_dtype, i));
    }
}

__global__ void block_table_lookup_kernel(const int32_t* __restrict__ bt, const int32_t* __restrict__ pos,
                                          int32_t* __restrict__ page_ids, int32_t* __restrict__ offsets, int B,
                                          int max_blocks, int page_size) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int p = pos[b];
    int blk = p / page_size;
    blk = max(0, min(blk, max_blocks - 1));   // callers range-check positions; the clamp only guards the load
    page_ids[b] = bt[(int64_t)b * max_blocks + blk];
    offsets[b] = p % page_size;
}

inline int grid_for(int64_t items, int threads) {
    const int64_t blocks = (items + threads - 1) / threads;
    const int64_t cap = (int64_t)sm_count() * 16;
    return (int)std::max<int64_t>(1, std::min(blocks, cap));
}

}  // namespace

int rmsnorm_residual_launch(const void* x, const void* residual, const void* weight, void* y, void* z_out,
                            int64_t rows, int64_t D, float eps, int dtype, int w_dtype, cudaStream_t stream) {
    if (dtype == B200Q_F16)
        rmsnorm_residual_kernel<__half><<<(unsigned)rows, 256, 0, stream>>>(
            (const __half*)x, (const __half*)residual, weight, (__half*)y, (__half*)z_out, D, eps, w_dtype);
    else
        rmsnorm_residual_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, stream>>>(
            (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, weight, (__nv_bfloat16*)y, (__nv_bfloat16*)z_out, D,
            eps, w_dtype);
    return finish_launch();
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_version(void) { return 100; }

const char* b200q_strerror(int code) {
    switch (code) {
        case B200Q_OK: return "ok";
        case B200Q_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size, unknown dtype or bits)";
        case B200Q_ERR_UNSUPPORTED: return "shape not supported by the CUDA kernels";
        case B200Q_ERR_LAUNCH: return "CUDA launch or runtime call failed";
        case B200Q_ERR_WORKSPACE: return "workspace missing or too small";
        case B200Q_ERR_DEVICE_WAIT: return "a bounded device-side wait gave up";
        case B200Q_ERR_STATIC_SCRATCH:
            return "problem too large for the library's built-in scratch array (see b200q_paged_gqa_static_scratch_bytes); "
                   "use b200q_paged_gqa_decode with a caller-allocated workspace";
        default: return "unknown b200q error";
    }
}

int b200q_device_status(int reset, void* stream) {
    const int a = gemv_read_status(reset, (cudaStream_t)stream);
    const int b = attn_read_status(reset, (cudaStream_t)stream);
    const int c = peer_read_status(reset, (cudaStream_t)stream);
    const int d = stack_read_status(reset, (cudaStream_t)stream);
    if (a < 0) return a;
    if (b < 0) return b;
    if (c < 0) return c;
    if (d < 0) return d;
    return std::max(std::max(a, b), std::max(c, d));
}

int b200q_peer_allgather(const void* local, void* const* peer_full, uint32_t* const* peer_flags, uint32_t* epoch,
                         int rank, int world, int rows, int64_t row_bytes_local, void* stream) {
    tp_discard();
    return peer_allgather_impl(local, peer_full, peer_flags, epoch, rank, world, rows, row_bytes_local,
                               (cudaStream_t)stream);
}

int b200q_wait_expiry_selftest(unsigned limit, uint32_t* probes_out, void* stream) {
    tp_discard();
    return wait_expiry_selftest_impl(limit, probes_out, (cudaStream_t)stream);
}

int b200q_tp_register(int slot, void* const* peer_full, uint32_t* const* peer_flags, uint32_t* epoch, uint32_t* counter,
                      int rank, int world) {
    if (slot < 0 || slot >= 16 || peer_full == nullptr || peer_flags == nullptr || epoch == nullptr || counter == nullptr)
        return B200Q_ERR_BAD_ARG;
    if (world < 2 || world > kTpMaxRanks || rank < 0 || rank >= world) return B200Q_ERR_BAD_ARG;
    TpSlot t = {};
    for (int r = 0; r < world; ++r) {
        if (peer_full[r] == nullptr || peer_flags[r] == nullptr) return B200Q_ERR_BAD_ARG;
        t.out.full[r] = peer_full[r];
        t.out.flags[r] = peer_flags[r];
    }
    t.out.epoch = epoch;
    t.out.counter = counter;
    t.out.rank = rank;
    t.out.world = world;
    std::lock_guard<std::mutex> lock(g_mu);
    g_tp_slots[slot] = t;
    g_tp_valid[slot] = true;
    return B200Q_OK;
}

int b200q_tp_set_packets(int slot, int packets) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (slot < 0 || slot >= 16 || !g_tp_valid[slot]) return B200Q_ERR_BAD_ARG;
    g_tp_slots[slot].out.packets = packets ? 1 : 0;
    return B200Q_OK;
}

int b200q_tp_next(int in_slot, int out_slot) {
    if ((in_slot >= 0 && tp_slot(in_slot) == nullptr) || (out_slot >= 0 && tp_slot(out_slot) == nullptr))
        return B200Q_ERR_BAD_ARG;
    g_tp_next_in = in_slot;
    g_tp_next_out = out_slot;
    return B200Q_OK;
}

int b200q_set_tuning(const char* key, int value) {
    if (key == nullptr) return B200Q_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(g_mu);
    g_tuning[key] = value;
    return B200Q_OK;
}

int b200q_dequant(int bits, const uint8_t* codes, const void* scales, const void* zeros, void* out, int64_t M,
                  int64_t K, int group_size, int scale_dtype, int out_dtype, void* stream) {
    tp_discard();
    if ((bits != 4 && bits != 8) || codes == nullptr || scales == nullptr || out == nullptr) return B200Q_ERR_BAD_ARG;
    if (M <= 0 || K <= 0 || group_size <= 0 || !is_scale_dtype(scale_dtype) || !is_act_dtype(out_dtype))
        return B200Q_ERR_BAD_ARG;
    const int64_t row_bytes = bits == 4 ? (K + 1) / 2 : K;
    const int Gn = (int)((K + group_size - 1) / group_size);
    const bool vec_ok = (K % 8 == 0) && ((uintptr_t)codes % 8 == 0) && ((uintptr_t)out % 16 == 0) && (row_bytes % 8 == 0);
    const int grid = grid_for(M * ((K + 7) / 8), 256);
    if (out_dtype == B200Q_F16)
        dequant_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>(bits, codes, scales, zeros, (__half*)out, M, K,
                                                                      group_size, Gn, row_bytes, scale_dtype, vec_ok);
    else
        dequant_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
            bits, codes, scales, zeros, (__nv_bfloat16*)out, M, K, group_size, Gn, row_bytes, scale_dtype, vec_ok);
    return finish_launch();
}

int b200q_qmatvec(int bits, const void* x, const uint8_t* codes, const void* scales, const void* zeros,
                  const void* residual, void* y, int B, int64_t N, int64_t K, int group_size, int act_dtype,
                  int scale_dtype, void* stream) {
    return qmatvec_impl(bits, x, codes, scales, zeros, residual, y, B, N, K, group_size, act_dtype, scale_dtype,
                        nullptr, nullptr, B200Q_F16, 0.0f, nullptr, nullptr, (cudaStream_t)stream);
}

int b200q_norm_qmatvec(int bits, const void* x, const void* residual_in, const void* norm_weight, int norm_w_dtype,
                       float eps, void* z_out, void* normed_out, const uint8_t* codes, const void* scales,
                       const void* zeros, const void* residual, void* y, int B, int64_t N, int64_t K, int group_size,
                       int act_dtype, int scale_dtype, void* stream) {
    if (norm_weight == nullptr) {
        tp_discard();
        return B200Q_ERR_BAD_ARG;
    }
    return qmatvec_impl(bits, x, codes, scales, zeros, residual, y, B, N, K, group_size, act_dtype, scale_dtype,
                        residual_in, norm_weight, norm_w_dtype, eps, z_out, normed_out, (cudaStream_t)stream);
}

int b200q_rope_kv_append(const void* qkv, const float* cos_table, const float* sin_table, const int32_t* positions,
                         const int32_t* block_table, void* q_out, uint8_t* k_codes, uint8_t* v_codes, void* k_scales,
                         void* v_scales, int bits, int B, int Hq, int Hkv, int D, int page_size, int64_t num_pages,
                         int max_blocks, int group_size, int table_len, void* stream) {
    tp_discard();
    return rope_kv_append_impl(qkv, cos_table, sin_table, positions, block_table, q_out, k_codes, v_codes, k_scales,
                               v_scales, bits, B, Hq, Hkv, D, page_size, num_pages, max_blocks, group_size, table_len,
                               (cudaStream_t)stream);
}

int b200q_gate_up_swiglu(int bits, const void* x, const uint8_t* gate_codes, const uint8_t* up_codes,
                         const void* gate_scales, const void* up_scales, const void* gate_zeros, const void* up_zeros,
                         void* gate_out, void* up_out, void* act_out, const void* residual_in, const void* norm_weight,
                         int norm_w_dtype, float eps, void* z_out, void* normed_out, int rows, int64_t N, int64_t K,
                         int group_size, int act_dtype, int scale_dtype, void* stream) {
    return gate_up_impl(bits, x, gate_codes, up_codes, gate_scales, up_scales, gate_zeros, up_zeros, gate_out, up_out,
                        act_out, residual_in, norm_weight, eps, z_out, normed_out, rows, N, K, group_size, act_dtype,
                        scale_dtype, norm_w_dtype, (cudaStream_t)stream);
}

int b200q_swiglu(const void* gate, const void* up, void* out, int64_t rows, int64_t dim, int dtype, void* stream) {
    tp_discard();
    if (gate == nullptr || up == nullptr || out == nullptr || rows <= 0 || dim <= 0 || !is_act_dtype(dtype))
        return B200Q_ERR_BAD_ARG;
    const int64_t n = rows * dim;
    const int grid = grid_for(n, 256);
    if (dtype == B200Q_F16)
        swiglu_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half*)gate, (const __half*)up, (__half*)out, n);
    else
        swiglu_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (__nv_bfloat16*)out, n);
    return finish_launch();
}

int b200q_residual_add(const void* x, const void* residual, void* out, int64_t n, int dtype, void* stream) {
    tp_discard();
    if (x == nullptr || residual == nullptr || out == nullptr || n <= 0 || !is_act_dtype(dtype)) return B200Q_ERR_BAD_ARG;
    const int grid = grid_for(n, 256);
    if (dtype == B200Q_F16)
        residual_add_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half*)x, (const __half*)residual,
                                                                           (__half*)out, n);
    else
        residual_add_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, n);
    return finish_launch();
}

int b200q_rmsnorm_residual(const void* x, const void* residual, const void* weight, void* y, void* z_out, int64_t rows,
                           int64_t D, float eps, int dtype, int w_dtype, void* stream) {
    tp_discard();
    if (x == nullptr || weight == nullptr || y == nullptr || rows <= 0 || D <= 0 || !is_act_dtype(dtype) ||
        !is_scale_dtype(w_dtype))
        return B200Q_ERR_BAD_ARG;
    return rmsnorm_residual_launch(x, residual, weight, y, z_out, rows, D, eps, dtype, w_dtype, (cudaStream_t)stream);
}

int b200q_block_table_lookup(const int32_t* block_table, const int32_t* positions, int32_t* page_ids, int32_t* offsets,
                             int B, int max_blocks, int page_size, void* stream) {
    tp_discard();
    if (block_table == nullptr || positions == nullptr || page_ids == nullptr || offsets == nullptr || B <= 0 ||
        max_blocks <= 0 || page_size <= 0)
        return B200Q_ERR_BAD_ARG;
    block_table_lookup_kernel<<<(B + 127) / 128, 128, 0, (cudaStream_t)stream>>>(block_table, positions, page_ids,
                                                                                 offsets, B, max_blocks, page_size);
    return finish_launch();
}

int b200q_attention_stage_launches(int B, int Hkv, int with_append) { return attention_stage_launches_impl(B, Hkv, with_append); }

size_t b200q_paged_gqa_workspace_bytes(int B, int Hq, int Hkv, int D) { return paged_gqa_workspace_bytes_impl(B, Hq, Hkv, D); }

int b200q_paged_gqa_decode(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                           const void* k_scales, const void* v_scales, const int32_t* block_table,
                           const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes, int B, int Hq,
                           int Hkv, int D, int page_size, int64_t num_pages, int max_blocks, int group_size, float scale,
                           int q_dtype, int scale_dtype, void* stream) {
    return paged_gqa_decode_impl(bits, q, k_codes, v_codes, k_scales, v_scales, block_table, lengths, out, workspace,
                                 workspace_bytes, B, Hq, Hkv, D, page_size, num_pages, max_blocks, group_size, scale,
                                 q_dtype, scale_dtype, 0, 0, (cudaStream_t)stream);
}

int b200q_paged_gqa_decode_window(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                                  const void* k_scales, const void* v_scales, const int32_t* block_table,
                                  const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes, int B,
                                  int Hq, int Hkv, int D, int page_size, int64_t num_pages, int max_blocks,
                                  int group_size, float scale, int q_dtype, int scale_dtype, int sink_tokens,
                                  int window_size, void* stream) {
    if (window_size <= 0) return B200Q_ERR_BAD_ARG;
    return paged_gqa_decode_impl(bits, q, k_codes, v_codes, k_scales, v_scales, block_table, lengths, out, workspace,
                                 workspace_bytes, B, Hq, Hkv, D, page_size, num_pages, max_blocks, group_size, scale,
                                 q_dtype, scale_dtype, sink_tokens, window_size, (cudaStream_t)stream);
}

int b200q_paged_gqa_decode_block_sparse(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                                        const void* k_scales, const void* v_scales, const int32_t* block_table,
                                        const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes,
                                        const uint8_t* block_mask, int n_qblocks, int n_kblocks, int block_size,
                                        int32_t* page_scratch, int B, int Hq, int Hkv, int D, int page_size,
                                        int64_t num_pages, int max_blocks, int group_size, float scale, int q_dtype,
                                        int scale_dtype, void* stream) {
    return paged_gqa_decode_block_sparse_impl(bits, q, k_codes, v_codes, k_scales, v_scales, block_table, lengths, out,
                                              workspace, workspace_bytes, block_mask, n_qblocks, n_kblocks, block_size,
                                              page_scratch, B, Hq, Hkv, D, page_size, num_pages, max_blocks, group_size,
                                              scale, q_dtype, scale_dtype, (cudaStream_t)stream);
}

size_t b200q_paged_fp16_gqa_workspace_bytes(int B, int Hq, int Hkv, int max_blocks) {
    return paged_fp16_workspace_bytes_impl(B, Hq, Hkv, max_blocks);
}

int b200q_paged_fp16_gqa_decode(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_table,
                                const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes, int B, int Hq,
                                int Hkv, int D, int page_size, int64_t num_pages, int max_blocks, float scale, int dtype,
                                void* stream) {
    tp_discard();
    return paged_fp16_gqa_decode_impl(q, k_pages, v_pages, block_table, lengths, out, workspace, workspace_bytes, B, Hq,
                                      Hkv, D, page_size, num_pages, max_blocks, scale, dtype, (cudaStream_t)stream);
}

int b200q_quantize_kv(int bits, const void* values, uint8_t* codes, void* scales, int64_t rows, int D, int group_size,
                      int in_dtype, void* stream) {
    tp_discard();
    return quantize_kv_impl(bits, values, codes, scales, rows, D, group_size, in_dtype, (cudaStream_t)stream);
}

int b200q_rope_append_paged_gqa_decode(const void* qkv, const float* cos_table, const float* sin_table,
                                       const int32_t* positions, int table_len, int bits, uint8_t* k_codes, uint8_t* v_codes,
                                       void* k_scales, void* v_scales, const int32_t* block_table, const int32_t* lengths,
                                       void* out, void* q_scratch, void* workspace, size_t workspace_bytes, int B, int Hq,
                                       int Hkv, int D, int page_size, int64_t num_pages, int max_blocks, int group_size,
                                       float scale, void* stream) {
    return rope_append_attention_impl(qkv, cos_table, sin_table, positions, table_len, bits, k_codes, v_codes, k_scales,
                                      v_scales, block_table, lengths, out, q_scratch, workspace, workspace_bytes, B, Hq, Hkv, D,
                                      page_size, num_pages, max_blocks, group_size, scale, (cudaStream_t)stream);
}

size_t b200q_paged_gqa_static_scratch_bytes(void) { return paged_gqa_static_scratch_bytes_impl(); }

int b200q_paged_gqa_decode_static(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                                  const void* k_scales, const void* v_scales, const int32_t* block_table,
                                  const int32_t* lengths, void* out, int B, int Hq, int Hkv, int D, int page_size,
                                  int64_t num_pages, int max_blocks, int group_size, float scale, int q_dtype,
                                  int scale_dtype, void* stream) {
    return paged_gqa_decode_static_impl(bits, q, k_codes, v_codes, k_scales, v_scales, block_table, lengths, out, B, Hq,
                                        Hkv, D, page_size, num_pages, max_blocks, group_size, scale, q_dtype, scale_dtype,
                                        (cudaStream_t)stream);
}

}  // extern "C"
