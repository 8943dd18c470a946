// Sum of a few floats over the GPUs of one node through peer memory (NVLink / NVSwitch), for the one collective of the
// data-parallel layers: the all-reduce of the learned-scalar gradients (lambda for TV; two alphas for TGV; 49 weights
// for the median filter).  At this size a collective is pure latency, so the exchange is one-shot: every rank stores its
// values straight into every peer's exchange buffer and then reads the values the peers stored into its own.
//
// Protocol.  A value travels with its call number in ONE naturally aligned 8-byte store (low word = the float's bits,
// high word = the call number), so no separate flag and no fence is needed: whoever sees the call number sees the
// value.  Each rank's buffer has two sets of world x 64 slots, used alternately by call number parity; a rank cannot
// be two calls ahead of a peer (it needs that peer's contribution to finish a call), so two sets are enough.  The sum
// is taken in rank order on every rank, which makes the result identical everywhere and independent of timing.
// Every wait is bounded: after about a second of polling the thread gives up, the result is NaN and the call number
// is written to a status word that cnl_peer_allreduce_status() returns.
#include "common.h"

namespace cnl {

constexpr int kPeerMaxCount = 64;
constexpr int kPeerMaxWorld = 16;
constexpr long long kPeerSpinLimit = 1ll << 22;

struct PeerBufs {
    unsigned long long* buf[kPeerMaxWorld];       // buf[r]: rank r's exchange buffer, as mapped into this process
};

__device__ int g_peer_status = 0;                  // call number of the last exchange that gave up, 0 if none

__device__ __forceinline__ size_t peer_slot(unsigned seq, int from_rank, int i) {
    return ((size_t)(seq & 1u) * kPeerMaxWorld + from_rank) * kPeerMaxCount + i;
}

// Exchanges v (element i of the vector) with all ranks and returns the sum in rank order.
__device__ __forceinline__ float peer_sum(float v, int i, const PeerBufs& pb, int rank, int world, unsigned seq) {
    const unsigned long long packed = ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(v);
    for (int r = 0; r < world; ++r) {
        volatile unsigned long long* dst = pb.buf[r] + peer_slot(seq, rank, i);
        *dst = packed;
    }
    float sum = 0.0f;
    bool gave_up = false;
    for (int r = 0; r < world; ++r) {
        const volatile unsigned long long* src = pb.buf[rank] + peer_slot(seq, r, i);
        unsigned long long got = *src;
        for (long long spin = 0; (unsigned)(got >> 32) != seq; ++spin) {
            if (spin >= kPeerSpinLimit) { gave_up = true; break; }
            __nanosleep(32);
            got = *src;
        }
        sum += __uint_as_float((unsigned)got);
    }
    if (gave_up) {
        g_peer_status = (int)seq;
        return __int_as_float(0x7fc00000);
    }
    return sum;
}

__global__ void __launch_bounds__(kPeerMaxCount)
peer_allreduce_kernel(float* __restrict__ values, int count, PeerBufs pb, int rank, int world, unsigned seq) {
    const int i = threadIdx.x;
    if (i < count) values[i] = peer_sum(values[i], i, pb, rank, world, seq);
}

// tv_dot_final_kernel with the exchange appended: the local sum never leaves the kernel before it is a global one.
__global__ void __launch_bounds__(32)
tv_dot_final_allreduce_kernel(const float* __restrict__ partial, int nblocks, float* __restrict__ out, PeerBufs pb,
                              int rank, int world, unsigned seq) {
    const double* p = reinterpret_cast<const double*>(partial);
    double s = 0.0;
    for (int i = threadIdx.x; i < nblocks; i += 32) s += p[i];
    for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
    if (threadIdx.x == 0) out[0] = peer_sum((float)s, 0, pb, rank, world, seq);
}

static int fill_bufs(PeerBufs& pb, void* const* peer_bufs, int rank, int world) {
    if (!peer_bufs) return fail(CNL_ERR_NULL, "null pointer argument");
    if (world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world)
        return fail(CNL_ERR_BAD_SHAPE, "rank %d / world %d is outside 1..%d ranks", rank, world, kPeerMaxWorld);
    for (int r = 0; r < kPeerMaxWorld; ++r) pb.buf[r] = nullptr;
    for (int r = 0; r < world; ++r) {
        if (!peer_bufs[r] || (reinterpret_cast<size_t>(peer_bufs[r]) & 7) != 0)
            return fail(CNL_ERR_NULL, "exchange buffer of rank %d is null or not 8-byte aligned", r);
        pb.buf[r] = static_cast<unsigned long long*>(peer_bufs[r]);
    }
    return CNL_OK;
}

int launch_tv_dot_final_allreduce(const float* partial, int nblocks, float* out, void* const* peer_bufs, int rank, int world,
                                  unsigned long long seq, cudaStream_t st) {
    PeerBufs pb;
    CNL_TRY(fill_bufs(pb, peer_bufs, rank, world));
    if (seq == 0) return fail(CNL_ERR_BAD_SHAPE, "call numbers start at 1 (the buffers start zeroed)");
    tv_dot_final_allreduce_kernel<<<1, 32, 0, st>>>(partial, nblocks, out, pb, rank, world, (unsigned)seq);
    return after_launch("tv_dot_final_allreduce_kernel");
}

}  // namespace cnl

using namespace cnl;

extern "C" long long cnl_peer_allreduce_bytes(void) {
    return 2ll * kPeerMaxWorld * kPeerMaxCount * (long long)sizeof(unsigned long long);
}

extern "C" int cnl_peer_allreduce_sum(float* values, int count, void* const* peer_bufs, int rank, int world,
                                      unsigned long long seq, void* stream) {
    if (!values) return fail(CNL_ERR_NULL, "null pointer argument");
    if (count < 0 || count > kPeerMaxCount) return fail(CNL_ERR_BAD_SHAPE, "at most %d values per call (got %d)", kPeerMaxCount, count);
    if (seq == 0) return fail(CNL_ERR_BAD_SHAPE, "call numbers start at 1 (the buffers start zeroed)");
    PeerBufs pb;
    CNL_TRY(fill_bufs(pb, peer_bufs, rank, world));
    if (count == 0) return CNL_OK;
    peer_allreduce_kernel<<<1, kPeerMaxCount, 0, static_cast<cudaStream_t>(stream)>>>(values, count, pb, rank, world, (unsigned)seq);
    return after_launch("peer_allreduce_kernel");
}

extern "C" int cnl_peer_allreduce_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_peer_status, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
    return v;
}
