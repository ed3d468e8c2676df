// Shared device/host helpers for libb200q (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200q.h"

namespace b200q {

// ---------------------------------------------------------------------------------------------
// Device status word: set by a kernel whose bounded wait ran out.  Each translation unit with
// waiting kernels owns one (B200Q_DEFINE_STATUS_WORD) and exports a host reader; the public
// b200q_device_status() takes the maximum over them.
// ---------------------------------------------------------------------------------------------
#define B200Q_DEFINE_STATUS_WORD(READER)                                                        \
    namespace {                                                                                 \
    __device__ int g_device_status = 0;                                                         \
    }                                                                                           \
    int READER(int reset, cudaStream_t stream) {                                                \
        int v = 0;                                                                              \
        if (cudaStreamSynchronize(stream) != cudaSuccess) return B200Q_ERR_LAUNCH;              \
        if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess)              \
            return B200Q_ERR_LAUNCH;                                                            \
        if (reset && v != 0) {                                                                  \
            const int zero = 0;                                                                 \
            if (cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)) != cudaSuccess)         \
                return B200Q_ERR_LAUNCH;                                                        \
        }                                                                                       \
        return v;                                                                               \
    }

enum DeviceEvent : int {
    EV_NONE = 0,
    EV_GEMV_FULL_WAIT = 1,    // consumer gave up waiting for a weight stage
    EV_GEMV_EMPTY_WAIT = 2,   // producer gave up waiting for a free stage
    EV_ATTN_FULL_WAIT = 3,
    EV_ATTN_EMPTY_WAIT = 4,
    EV_PEER_WAIT = 5,         // a rank gave up waiting for a peer's shard in the peer all-gather
    EV_ROPE_POSITION = 6,     // rope + append: a position lies outside the rotary table (row left unrotated)
    EV_KV_PAGE_UNASSIGNED = 7,  // rope + append: the block table has no page for the position (nothing appended)
};

// ---------------------------------------------------------------------------------------------
// Tensor-parallel exchange fused into kernels (see b200q_tp_register / b200q_tp_next).  The writer kernel
// stores its output rows into column block `rank` of every rank's full buffer [rows, world * n] (peer stores)
// and its last CTA publishes a sequence number in every rank's flag word; the reader kernel waits, bounded,
// until the flag words of all source ranks carry the sequence number of its own rank's latest publication.
// ---------------------------------------------------------------------------------------------
constexpr int kTpMaxRanks = 8;
struct TpOut {
    void* full[kTpMaxRanks];        // full buffer of rank r as mapped on this GPU
    uint32_t* flags[kTpMaxRanks];   // flag words [world] of rank r as mapped on this GPU
    uint32_t* epoch;                // this rank's publication counter for the buffer (device memory)
    uint32_t* counter;              // CTAs of the writer kernel that have finished (device memory, zero between uses)
    int rank, world;                // world == 0: no exchange
    int packets;                    // 1: the full buffers hold 4-byte packets (16 data bits + 16 sequence bits) instead of
                                    // plain 16-bit rows, and no flag words are used (see tp_packet below)
};
struct TpIn {
    const uint32_t* flags;          // this rank's flag words [world]
    const uint32_t* epoch;          // this rank's publication counter (already advanced by the local writer)
    int world;                      // world == 0: nothing to wait for
    uint32_t spin_limit;            // acquire loads before the wait gives up (0: kTpSpinLimit); tuning key "tp.spin_limit"
    int packets;                    // 1: the activations are a packet buffer; every load checks its own packets
};
struct TpSlot { TpOut out; };       // host table entry
const TpSlot* tp_slot(int slot);    // nullptr if the slot was never registered
void tp_take(int* in_slot, int* out_slot);   // exchange slots set by b200q_tp_next for the next call (then cleared)
void tp_discard();                           // entry points without an exchange drop a pending request

// ---------------------------------------------------------------------------------------------
// Tuning table (host side; see b200q_set_tuning)
// ---------------------------------------------------------------------------------------------
int tuning_get(const char* key);

int sm_count();          // multiprocessors of the current device (cached per device)
int max_smem_optin();    // opt-in shared memory per block of the current device

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: spins at most `limit` probes (each probe itself blocks for a hardware-defined
// short time).  On expiry the event code is recorded in the status word and false is returned;
// the caller carries on without the data so that the kernel still terminates.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* status_word, int event,
                                                  uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    atomicMax(status_word, event);
    return false;
}

// 1-D bulk copy global -> shared, completion signalled on an mbarrier (TMA engine, no tensor map).
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Programmatic dependent launch.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
constexpr uint32_t kTpSpinLimit = 1u << 22;   // acquire loads; each takes a fraction of a microsecond
// Called by one whole warp of every CTA of the writer kernel after its stores: the last CTA publishes.
__device__ __forceinline__ void tp_finish_writer(const TpOut& out, int lane, unsigned total_ctas = 0) {
    if (total_ctas == 0) total_ctas = gridDim.x * gridDim.y;
    __threadfence_system();                      // this CTA's peer stores are visible before it is counted
    __syncwarp();
    unsigned last = 0;
    if (lane == 0) last = (atomicAdd(out.counter, 1u) == total_ctas - 1u) ? 1u : 0u;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
        __threadfence_system();
        const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(out.epoch) + 1u;
        if (lane < out.world) st_release_sys(out.flags[lane] + out.rank, seq);
        __syncwarp();
        if (lane == 0) {
            *out.epoch = seq;
            *out.counter = 0u;
        }
    }
}
// Called by threads 0 .. world-1 of the reader; returns false when the bounded wait ran out.
__device__ __forceinline__ bool tp_wait_source(const TpIn& in, int src) {
    const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(in.epoch);
    const uint32_t limit = in.spin_limit ? in.spin_limit : kTpSpinLimit;
    for (uint32_t it = 0; it < limit; ++it)
        if ((int32_t)(ld_acquire_sys(in.flags + src) - seq) >= 0) return true;
    return false;
}

// ---- packet form of the exchange: payload and "it has arrived" in ONE 4-byte store ----------------------------
// A full buffer in packet form holds one 32-bit word per 16-bit element: the element in the low half, the low bits of
// the exchange's sequence number (never 0; the buffers start zeroed) in the high half.  A 4-byte store is single-copy
// atomic, so a reader that finds the expected sequence number has the element - no fence, no flag word, no counter
// round trip across NVLink: an exchange costs one one-way store latency instead of a fence round trip plus a flag.
// Every exchange rewrites all packets of its buffer, so a stale packet carries the previous sequence number.
__device__ __forceinline__ uint32_t tp_seq16(uint32_t seq) { return seq % 65535u + 1u; }
__device__ __forceinline__ uint32_t tp_packet(unsigned short bits16, uint32_t seq16) { return (uint32_t)bits16 | (seq16 << 16); }
__device__ __forceinline__ void st_volatile_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_u128(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// Sequence number the writer kernel stamps its packets with; read after griddepcontrol.wait (everything earlier in the
// stream, the previous use of the buffer included, is complete then).
__device__ __forceinline__ uint32_t tp_writer_seq(const TpOut& out) {
    return *reinterpret_cast<const volatile uint32_t*>(out.epoch) + 1u;
}
// Called by one whole warp of every CTA of the writer kernel after its packet stores: the last CTA advances this
// rank's sequence counter (local memory only: the packets need no publication).
__device__ __forceinline__ void tp_finish_writer_packets(const TpOut& out, int lane, unsigned total_ctas = 0) {
    if (total_ctas == 0) total_ctas = gridDim.x * gridDim.y;
    __syncwarp();
    if (lane == 0) {
        __threadfence();
        if (atomicAdd(out.counter, 1u) == total_ctas - 1u) {
            const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(out.epoch) + 1u;
            *out.epoch = seq;
            *out.counter = 0u;
        }
    }
}
// 8 consecutive elements (32 bytes of packets, 32-byte aligned) of a packet buffer; polls until all eight carry
// `seq16`, at most `limit` times.  Returns false when the wait ran out (the data are then whatever was there).
__device__ __forceinline__ bool tp_load8_packets(const void* base, int64_t idx, uint32_t seq16, uint32_t limit, uint32_t (&w)[4]) {
    const char* src = reinterpret_cast<const char*>(base) + idx * 4;
    const uint32_t want = seq16 << 16;
    uint4 a, b;
    bool ok = false;
    for (uint32_t it = 0; it < limit; ++it) {
        a = ld_volatile_u128(src);
        b = ld_volatile_u128(src + 16);
        const uint32_t diff = ((a.x ^ want) | (a.y ^ want) | (a.z ^ want) | (a.w ^ want) |
                               (b.x ^ want) | (b.y ^ want) | (b.z ^ want) | (b.w ^ want)) & 0xFFFF0000u;
        if (diff == 0u) { ok = true; break; }
    }
    w[0] = (a.x & 0xFFFFu) | (a.y << 16);
    w[1] = (a.z & 0xFFFFu) | (a.w << 16);
    w[2] = (b.x & 0xFFFFu) | (b.y << 16);
    w[3] = (b.z & 0xFFFFu) | (b.w << 16);
    return ok;
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));   // (a & b) | c
    return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
// Transposes an 8x8 matrix of 16-bit values held one row per 4 lanes (lane l: row l/4, columns 2(l%4), 2(l%4)+1).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(a));
    return r;
}
__device__ __forceinline__ uint32_t half_dup(__half h) {
    uint32_t u = __half_as_ushort(h);
    return u | (u << 16);
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------------------------
// In-register dequantisation: packed codes -> fp16(code * scale), two values per register.
//
// q4: a 32-bit word holds nibbles n0..n7 (n0 lowest).  OR-ing a nibble into the mantissa of
// 1024.0 (bits 0-3) or of 64.0 (bits 4-7) gives the exact halves 1024+n / 64+n; one fused
// multiply-add with (s, -1024 s) or (s, -64 s) then yields n*s with a single rounding, because
// 1024 s and 64 s are exact in fp16.  Output order: (n0,n4) (n1,n5) (n2,n6) (n3,n7).
// ---------------------------------------------------------------------------------------------
struct ScaleRegs {
    uint32_t s2;      // (s, s)
    uint32_t c1024;   // (-1024 s, -1024 s)
    uint32_t c64;     // (-64 s, -64 s)
};
__device__ __forceinline__ ScaleRegs make_scale_regs(__half s) {
    ScaleRegs r;
    r.s2 = half_dup(s);
    r.c1024 = hmul2_u32(r.s2, 0xE400E400u);   // -1024.0
    r.c64 = hmul2_u32(r.s2, 0xD400D400u);     // -64.0
    return r;
}
__device__ __forceinline__ void dequant_q4_word(uint32_t w, const ScaleRegs& sc, uint32_t (&v)[4]) {
    const uint32_t w2 = w >> 8;
    v[0] = hfma2_u32(lop3_and_or(w, 0x000F000Fu, 0x64006400u), sc.s2, sc.c1024);
    v[1] = hfma2_u32(lop3_and_or(w, 0x00F000F0u, 0x54005400u), sc.s2, sc.c64);
    v[2] = hfma2_u32(lop3_and_or(w2, 0x000F000Fu, 0x64006400u), sc.s2, sc.c1024);
    v[3] = hfma2_u32(lop3_and_or(w2, 0x00F000F0u, 0x54005400u), sc.s2, sc.c64);
}
// q8: bytes b0..b3 -> (b0,b1) (b2,b3), each 1024+b via a byte permute with the magic 0x64.
__device__ __forceinline__ void dequant_q8_word(uint32_t w, const ScaleRegs& sc, uint32_t (&v)[2]) {
    v[0] = hfma2_u32(prmt(w, 0x64646464u, 0x4140u), sc.s2, sc.c1024);
    v[1] = hfma2_u32(prmt(w, 0x64646464u, 0x4342u), sc.s2, sc.c1024);
}

// ---------------------------------------------------------------------------------------------
// dtype helpers
// ---------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

// Largest finite value of the activation dtype (the reference clips matvec results to finfo
// before the cast, ops/quant_ops.py:525-526).
template <typename T> __device__ __forceinline__ float finite_max();
template <> __device__ __forceinline__ float finite_max<__half>() { return 65504.0f; }
template <> __device__ __forceinline__ float finite_max<__nv_bfloat16>() { return 3.3895313892515355e38f; }

__device__ __forceinline__ float load_as_f32(const void* p, int dtype, int64_t i) {
    if (dtype == B200Q_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
    if (dtype == B200Q_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    return reinterpret_cast<const float*>(p)[i];
}

inline int dtype_size(int dtype) { return dtype == B200Q_F32 ? 4 : 2; }
inline bool is_act_dtype(int dtype) { return dtype == B200Q_F16 || dtype == B200Q_BF16; }
inline bool is_scale_dtype(int dtype) { return dtype == B200Q_F16 || dtype == B200Q_BF16 || dtype == B200Q_F32; }

inline int finish_launch() { return cudaGetLastError() == cudaSuccess ? B200Q_OK : B200Q_ERR_LAUNCH; }

}  // namespace b200q
