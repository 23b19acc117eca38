// Tensor-parallel exchange of one token's activations by peer stores, in place of an NCCL all-gather.
//
// Every rank owns an exchange buffer of tagged pairs {value, tag} (two slots, used alternately) that its peers have
// mapped (CUDA IPC). One kernel per exchange and rank, a single CTA: it stores its own slice of the vector - value and
// tag in ONE 8-byte store each - straight into every rank's buffer over NVLink, then reads its own buffer until every
// pair carries the exchange's tag, and writes the plain vector for the kernels that follow. A pair is either the old one
// or the new one, never half of each, so no flag, fence or second round trip is needed; the tag is a counter in device
// memory that every rank advances once per exchange (so a replayed CUDA graph keeps counting), and since a rank can
// finish exchange k only after every peer has at least started pushing k, ranks are never more than one exchange apart:
// two slots are enough. Every wait is bounded: a rank whose peer never writes gives up, sets the error word the session
// reads after the call, and ends.
//
// Kernels of different ranks wait for one another here, which is only sound because every rank has its own GPU.
#include "kernels.h"

namespace bk {
namespace {

constexpr uint32_t kPeerThreads = 1024;
constexpr uint32_t kPeerPollLimit = 1u << 22;  // re-reads of one pair (~a second) before giving up

struct PeerParams {
    uint2* const* bufs;  // device array [tp]: every rank's exchange buffer, as mapped into this process
    uint32_t* epoch;     // the next exchange's tag
    unsigned int* error;
    const float* local;  // this rank's slice [rows_l]
    float* dst;          // the whole vector [rows_l * tp]
    uint32_t tp, rank, rows_l, slot_pairs;
    int add;
};

// One 64-bit scalar access per pair: single-copy atomic in the memory model (a two-element vector access is not), so a
// reader sees the old pair or the new one, never the new tag with the old value.
__device__ __forceinline__ void st_pair_sys(uint2* p, float v, uint32_t tag) {
    const unsigned long long w = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_pair_sys(const uint2* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return make_uint2(static_cast<uint32_t>(w), static_cast<uint32_t>(w >> 32));
}

__global__ void __launch_bounds__(kPeerThreads) tp_peer_exchange_kernel(const PeerParams p) {
    const uint32_t tid = threadIdx.x;
    // After a wait has run out the call is lost anyway (the host raises when it ends): the exchanges still queued behind it
    // return at once instead of each waiting out its own limit.
    if (*reinterpret_cast<volatile unsigned int*>(p.error) != 0) return;
    const uint32_t tag = *reinterpret_cast<volatile uint32_t*>(p.epoch);
    const uint32_t slot = (tag & 1u) * p.slot_pairs;
    uint2* peer[8];  // the ranks' buffers, read from the table once (tensor parallelism goes up to 8 ranks)
#pragma unroll
    for (uint32_t r = 0; r < 8; ++r) peer[r] = r < p.tp ? p.bufs[r] + slot + p.rank * p.rows_l : nullptr;
    for (uint32_t i = tid; i < p.rows_l; i += kPeerThreads) {
        const float v = p.local[i];
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) {
            if (r < p.tp) st_pair_sys(peer[r] + i, v, tag);
        }
    }
    const uint2* mine = p.bufs[p.rank] + slot;
    // Read back in batches of independent loads: one L2 round trip fetches a thread's whole share when it is already there
    // (one pair after the other, each round trip waited for the one before: 14 of them for the widest vector), and only
    // what has not arrived yet is read again.
    constexpr uint32_t kBatch = 8;
    const uint32_t total = p.rows_l * p.tp;
    bool dead = false;
    for (uint32_t j0 = tid; j0 < total; j0 += kBatch * kPeerThreads) {
        uint2 w[kBatch];
        uint32_t pending = 0;
#pragma unroll
        for (uint32_t k = 0; k < kBatch; ++k) {
            const uint32_t j = j0 + k * kPeerThreads;
            if (j < total) {
                w[k] = ld_pair_sys(mine + j);
                pending |= (w[k].y != tag) << k;
            } else {
                w[k] = make_uint2(0, tag);
            }
        }
        for (uint32_t spin = 0; pending != 0 && !dead; ++spin) {
            if (spin == kPeerPollLimit) {
                atomicOr(p.error, 1u);
                dead = true;
                break;
            }
#pragma unroll
            for (uint32_t k = 0; k < kBatch; ++k) {
                if (pending & (1u << k)) {
                    w[k] = ld_pair_sys(mine + j0 + k * kPeerThreads);
                    if (w[k].y == tag) pending &= ~(1u << k);
                }
            }
        }
#pragma unroll
        for (uint32_t k = 0; k < kBatch; ++k) {
            const uint32_t j = j0 + k * kPeerThreads;
            if (j < total && !(pending & (1u << k))) {
                const float v = __uint_as_float(w[k].x);
                p.dst[j] = p.add ? __fadd_rn(p.dst[j], v) : v;
            }
        }
    }
    __syncthreads();  // every thread has read the tag
    if (tid == 0) *p.epoch = tag + 1;
}

}  // namespace

void launch_tp_peer_exchange(uint2* const* bufs_dev, uint32_t* epoch, unsigned int* error, uint32_t tp, uint32_t rank, uint32_t slot_pairs,
                             const float* local, float* dst, uint32_t rows_l, bool add, cudaStream_t s) {
    PeerParams p{bufs_dev, epoch, error, local, dst, tp, rank, rows_l, slot_pairs, add ? 1 : 0};
    tp_peer_exchange_kernel<<<1, kPeerThreads, 0, s>>>(p);
    BK_CUDA(cudaGetLastError());
}

}  // namespace bk
