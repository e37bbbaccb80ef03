// Expert-parallel all-to-all over peer memory (NVLink / NVSwitch), fused with the routing bookkeeping.
//
// Tokens are sharded over the ranks; every rank owns E / world experts.  Slot s = token * top_k + k of a source
// rank has a fixed place in every destination's receive area, so no size exchange is needed:
//
//   ep_dispatch   one CTA per (token, k): stores the activation row into the owner rank's receive buffer
//                 [src][slot][H] (peer store) and the slot's local expert id into EVERY rank's id table
//                 [src][slot] (-1 where the slot is not for that rank, and for the unused tail of the step's slot
//                 stride); the last CTA publishes the rank's epoch.  The stride is per step (rows per rank x top_k).
//   ep_wait       bounded wait until every source rank has published the epoch (one tiny CTA).
//                 The receiving rank then runs moe_align / gather / grouped GEMMs over the id table as usual.
//   ep_return     one CTA per received slot with a valid expert: stores the expert output row back into the
//                 source rank's combine buffer [slot][H] (peer store); last CTA publishes.  After ep_wait the
//                 source rank reduces its top_k rows per token with the router weights (moe_combine).
//
// All spins are bounded and report through the status word.  Plain loads and stores only on peer memory.
// The reference has no expert parallelism (docs/source/user_guide/features/multi-device.md:10-11).
#include "host_utils.h"
#include "tc5_common.cuh"

namespace telb {

constexpr int kEpMaxRanks = 8;

struct EpPeers {
    void* recv_rows[kEpMaxRanks];     // every rank's receive buffer   [world][slots_cap][hidden] 16-bit
    int* recv_ids[kEpMaxRanks];       // every rank's id table         [world][slots_cap]
    void* comb_rows[kEpMaxRanks];     // every rank's combine buffer   [slots_cap][hidden] 16-bit
    int* flags[kEpMaxRanks];          // every rank's flags            [2][kEpMaxRanks]: dispatch epochs, return epochs
};

__device__ __forceinline__ void ep_st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ep_ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Last CTA of the grid: make every peer store of this kernel visible, then publish `epoch + 1` in slot
// flags[which][rank] of every rank and advance the local epoch.
__device__ __forceinline__ void ep_publish(const EpPeers& peers, int which, int rank, int world, int* epoch, int* ticket) {
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(ticket, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        const int e = *epoch + 1;
        if (threadIdx.x < world) ep_st_release_sys(peers.flags[threadIdx.x] + which * kEpMaxRanks + rank, e);
        __syncthreads();
        if (threadIdx.x == 0) {
            *ticket = 0;
            *epoch = e;
        }
    }
}

// grid = slots_cap CTAs (the step's slot stride: every rank's segment of the id tables is rewritten in full, so no stale
// entry of an earlier, longer step survives); x [tokens_local, hidden] 16-bit; topk_idx [tokens_local, top_k] global expert ids.
__global__ void ep_dispatch_kernel(const uint4* __restrict__ x, const int* __restrict__ topk_idx, EpPeers peers, int rank, int world,
                                   int slots, int slots_cap, int top_k, int hidden, int experts_per_rank, int* epoch, int* ticket) {
    pdl_prologue();
    const int slot = blockIdx.x;
    if (slot < slots) {
        const int e = topk_idx[slot];
        const int dest = e / experts_per_rank;
        if (threadIdx.x < world) {
            const int id = (threadIdx.x == dest) ? e - dest * experts_per_rank : -1;
            peers.recv_ids[threadIdx.x][(size_t)rank * slots_cap + slot] = id;
        }
        const uint4* src = x + (size_t)(slot / top_k) * (hidden / 8);
        uint4* dst = reinterpret_cast<uint4*>(peers.recv_rows[dest]) + ((size_t)rank * slots_cap + slot) * (hidden / 8);
        for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
    } else if (slot < slots_cap && threadIdx.x < world) {
        peers.recv_ids[threadIdx.x][(size_t)rank * slots_cap + slot] = -1;      // unused tail of this rank's segment
    }
    ep_publish(peers, 0, rank, world, epoch, ticket);
}

// One CTA: wait until flags[which][src] >= *epoch for every source rank (epoch was advanced by this rank's own publish).
__global__ void ep_wait_kernel(const int* __restrict__ flags, int which, int world, const int* __restrict__ epoch, int* status) {
    pdl_prologue();
    if (threadIdx.x < world) {
        const int e = *epoch;
        const long long c0 = clock64();
        uint32_t it = 0;
        while (ep_ld_acquire_sys(flags + which * kEpMaxRanks + threadIdx.x) - e < 0) {
            if ((++it & 255u) == 0 && clock64() - c0 > kSpinLimitCycles) {
                atomicCAS(status, kStatusOk, kStatusPeerTimeout);
                break;
            }
        }
    }
}

// grid = world * slots_cap received slots; y [rows_pad, hidden] expert outputs, dst_row [world * slots_cap] (from moe_align).
__global__ void ep_return_kernel(const uint4* __restrict__ y, const int* __restrict__ dst_row, EpPeers peers, int rank, int world,
                                 int slots_cap, int hidden, int* epoch, int* ticket) {
    pdl_prologue();
    const int rs = blockIdx.x;                      // received slot: source rank * slots_cap + slot
    const int row = dst_row[rs];
    if (row >= 0) {
        const int src = rs / slots_cap, slot = rs - src * slots_cap;
        const uint4* from = y + (size_t)row * (hidden / 8);
        uint4* to = reinterpret_cast<uint4*>(peers.comb_rows[src]) + (size_t)slot * (hidden / 8);
        for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) to[i] = from[i];
    }
    ep_publish(peers, 1, rank, world, epoch, ticket);
}

}  // namespace telb

using namespace telb;

static int fill_peers(EpPeers& p, void* const* recv_rows, int* const* recv_ids, void* const* comb_rows, int* const* flags, int world) {
    if (world < 1 || world > kEpMaxRanks) return fail("expert-parallel world size must be in [1, 8]");
    for (int r = 0; r < world; ++r) {
        p.recv_rows[r] = recv_rows[r];
        p.recv_ids[r] = recv_ids[r];
        p.comb_rows[r] = comb_rows[r];
        p.flags[r] = flags[r];
    }
    return 0;
}

// Pointer tables hold `world` peer mappings each.  `slots_stride` is the slot count every rank reserves per source rank in this
// step (the same number on every rank, e.g. rows-per-rank x top_k; at most the buffers' capacity): the receive areas are laid
// out [source][slots_stride], so the work of a step follows its size, not the capacity.
extern "C" int telb_ep_dispatch(const void* x, const int* topk_idx, void* const* recv_rows, int* const* recv_ids, void* const* comb_rows,
                                int* const* flags, int rank, int world, int tokens_local, int top_k, int hidden, int experts_per_rank,
                                int slots_stride, int* epoch, int* ticket, cudaStream_t stream) {
    const int slots = tokens_local * top_k;
    if (slots_stride < 1) return fail("telb_ep_dispatch: slot stride must be positive");
    if (slots > slots_stride) return fail("telb_ep_dispatch: more routed rows than the step's slot stride");
    if (hidden % 8) return fail("telb_ep_dispatch: hidden must be a multiple of 8");
    EpPeers p{};
    if (fill_peers(p, recv_rows, recv_ids, comb_rows, flags, world)) return -1;
    TELB_LAUNCH("ep_dispatch_kernel", ep_dispatch_kernel, dim3(slots_stride), dim3(128), 0, stream, (const uint4*)x, topk_idx, p, rank,
                world, slots, slots_stride, top_k, hidden, experts_per_rank, epoch, ticket);
    return 0;
}

extern "C" int telb_ep_wait(const int* flags, int which, int world, const int* epoch, int* status, cudaStream_t stream) {
    TELB_LAUNCH("ep_wait_kernel", ep_wait_kernel, dim3(1), dim3(32), 0, stream, flags, which, world, epoch, status);
    return 0;
}

extern "C" int telb_ep_return(const void* y, const int* dst_row, void* const* recv_rows, int* const* recv_ids, void* const* comb_rows,
                              int* const* flags, int rank, int world, int slots_cap, int hidden, int* epoch, int* ticket,
                              cudaStream_t stream) {
    EpPeers p{};
    if (fill_peers(p, recv_rows, recv_ids, comb_rows, flags, world)) return -1;
    TELB_LAUNCH("ep_return_kernel", ep_return_kernel, dim3(world * slots_cap), dim3(128), 0, stream, (const uint4*)y, dst_row, p, rank, world,
                slots_cap, hidden, epoch, ticket);
    return 0;
}
