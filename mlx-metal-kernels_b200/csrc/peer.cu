// All-gather of a small activation shard over NVLink peer memory, for the tensor-parallel decode stack.
//
// Every rank holds `local` [rows, n_loc] and a `full` buffer [rows, world * n_loc] that all ranks can
// address (symmetric memory: the same allocation mapped on every GPU).  One CTA per rank stores its shard
// into column block `rank` of every rank's `full` buffer with plain peer stores, publishes a sequence
// number in each peer's flag slot (release at system scope) and then waits, with a bound, until the flag
// slots of all source ranks show the same sequence number (acquire).  The shards are a few KB, so the
// exchange costs a few microseconds instead of a collective launch per gather.
//
// No TMA, no multicast: ordinary st.global / ld.global on mapped peer addresses only.
#include "common.cuh"

namespace b200q {

B200Q_DEFINE_STATUS_WORD(peer_read_status)

namespace {

constexpr int kMaxRanks = 8;
constexpr uint32_t kPeerSpinLimit = 1u << 22;   // acquire loads; each takes a fraction of a microsecond

struct PeerGatherParams {
    const uint4* local;                 // [rows, vec_loc] 16-byte vectors
    uint4* full[kMaxRanks];             // full buffer of rank r as seen from this GPU
    uint32_t* flags[kMaxRanks];         // flag array [world] of rank r as seen from this GPU
    uint32_t* epoch;                    // this rank's sequence counter for this buffer (device memory)
    int rank, world, rows, vec_loc;     // vec_loc = 16-byte vectors per row of the local shard
    uint32_t spin_limit;                // acquire loads before the wait gives up (tuning key "peer.spin_limit")
};

__global__ void __launch_bounds__(512) peer_allgather_kernel(const __grid_constant__ PeerGatherParams p) {
    const uint32_t seq = *p.epoch + 1u;             // identical on all ranks: every rank counts its own calls
    const int total = p.rows * p.vec_loc;
    const int vec_full = p.vec_loc * p.world;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int r = i / p.vec_loc;
        const int c = i - r * p.vec_loc;
        const uint4 v = p.local[i];
        const size_t dst = (size_t)r * vec_full + (size_t)p.rank * p.vec_loc + c;
#pragma unroll 1
        for (int peer = 0; peer < p.world; ++peer) p.full[peer][dst] = v;
    }
    __threadfence_system();                          // the stores above are visible before the flag
    __syncthreads();
    if ((int)threadIdx.x < p.world) {
        st_release_sys(p.flags[threadIdx.x] + p.rank, seq);
        // wait for source rank threadIdx.x; the sequence numbers only grow (wrap-around compared as signed distance)
        const uint32_t* mine = p.flags[p.rank] + threadIdx.x;
        bool seen = false;
        for (uint32_t it = 0; it < p.spin_limit; ++it) {
            if ((int32_t)(ld_acquire_sys(mine) - seq) >= 0) { seen = true; break; }
        }
        if (!seen) atomicMax(&g_device_status, (int)EV_PEER_WAIT);
    }
    __syncthreads();
    if (threadIdx.x == 0) *p.epoch = seq;
}

}  // namespace

int peer_allgather_impl(const void* local, void* const* peer_full, uint32_t* const* peer_flags, uint32_t* epoch,
                        int rank, int world, int rows, int64_t row_bytes_local, cudaStream_t stream) {
    if (local == nullptr || peer_full == nullptr || peer_flags == nullptr || epoch == nullptr) return B200Q_ERR_BAD_ARG;
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || rows <= 0 || row_bytes_local <= 0)
        return B200Q_ERR_BAD_ARG;
    if (row_bytes_local % 16 != 0 || (reinterpret_cast<uintptr_t>(local) & 15u) != 0) return B200Q_ERR_UNSUPPORTED;
    if (rows * (row_bytes_local / 16) > (int64_t)1 << 24) return B200Q_ERR_UNSUPPORTED;
    PeerGatherParams p = {};
    p.local = reinterpret_cast<const uint4*>(local);
    for (int r = 0; r < world; ++r) {
        if (peer_full[r] == nullptr || peer_flags[r] == nullptr) return B200Q_ERR_BAD_ARG;
        if ((reinterpret_cast<uintptr_t>(peer_full[r]) & 15u) != 0) return B200Q_ERR_UNSUPPORTED;
        p.full[r] = reinterpret_cast<uint4*>(peer_full[r]);
        p.flags[r] = peer_flags[r];
    }
    p.epoch = epoch;
    p.rank = rank; p.world = world; p.rows = rows; p.vec_loc = (int)(row_bytes_local / 16);
    const int limit = tuning_get("peer.spin_limit");
    p.spin_limit = limit > 0 ? (uint32_t)limit : kPeerSpinLimit;
    peer_allgather_kernel<<<1, 512, 0, stream>>>(p);
    return finish_launch();
}

// One CTA whose first thread waits, with the given bound, on an mbarrier that nothing ever arrives on: the wait runs
// out, EV_GEMV_FULL_WAIT is recorded in this unit's status word and the kernel returns.  It is the bounded-wait helper
// of the matvec and attention kernels run by itself, so that the give-up branch can be tested without making a
// product kernel lose a copy.
__global__ void wait_expiry_selftest_kernel(uint32_t limit, uint32_t* probes_out) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool got = mbar_wait_bounded(&bar, 0, &g_device_status, (int)EV_GEMV_FULL_WAIT, limit);
        if (probes_out != nullptr) *probes_out = got ? 0u : limit;
    }
}

int wait_expiry_selftest_impl(uint32_t limit, uint32_t* probes_out, cudaStream_t stream) {
    if (limit == 0 || limit > (1u << 16)) return B200Q_ERR_BAD_ARG;      // a test hook: short waits only
    wait_expiry_selftest_kernel<<<1, 32, 0, stream>>>(limit, probes_out);
    return finish_launch();
}

}  // namespace b200q
