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

// lambda gradient of the TV layer, out = sum a * b, in ONE launch, with the exchange appended where there are peers: the
// local sum never leaves the kernel before it is a global one.  Every block leaves its partial sum (a double) in the
// caller's scratch and takes a ticket; the block that draws the last ticket adds the partials in a fixed order, so the
// result does not depend on which block that was.  Tickets are words of a library-owned table that the last block
// resets to zero; every call takes the next word (the host counts), so calls that run side by side on different
// streams do not share one.
constexpr int kDotTickets = 4096;
__device__ unsigned int g_dot_tickets[kDotTickets];

template <bool kExchange>
__global__ void __launch_bounds__(256)
tv_dot_kernel(const float* __restrict__ a, const float* __restrict__ b, long long count, double* partial, float* __restrict__ out,
              int ticket, PeerBufs pb, int rank, int world, unsigned seq) {
    __shared__ double sh[8];
    __shared__ bool last;
    double s = 0.0;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
        s += (double)a[i] * (double)b[i];
    for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double ts = 0.0;
        for (int i = 0; i < 8; ++i) ts += sh[i];
        partial[blockIdx.x] = ts;
        __threadfence();                                        // the partial is visible before the ticket is
        last = atomicAdd(&g_dot_tickets[ticket], 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    double v = 0.0;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += 256) v += __ldcg(partial + i);
    for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        double ts = 0.0;
        for (int i = 0; i < 8; ++i) ts += sh[i];
        g_dot_tickets[ticket] = 0u;                             // ready for the call that takes this word next
        out[0] = kExchange ? peer_sum((float)ts, 0, pb, rank, world, seq) : (float)ts;
    }
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

int launch_tv_dot(const float* a, const float* b, long long count, float* out, float* scratch, int nblocks,
                  void* const* peer_bufs, int rank, int world, unsigned long long seq, cudaStream_t st) {
    static std::atomic<unsigned> next_ticket{0};
    const int ticket = (int)(next_ticket.fetch_add(1, std::memory_order_relaxed) % kDotTickets);
    double* partial = reinterpret_cast<double*>(scratch);
    PeerBufs pb;
    if (!peer_bufs) {
        for (int r = 0; r < kPeerMaxWorld; ++r) pb.buf[r] = nullptr;
        tv_dot_kernel<false><<<nblocks, 256, 0, st>>>(a, b, count, partial, out, ticket, pb, 0, 1, 0u);
        return after_launch("tv_dot_kernel");
    }
    CNL_TRY(fill_bufs(pb, peer_bufs, rank, world));
    if (seq == 0) return fail(CNL_ERR_BAD_SHAPE, "call numbers start at 1 (the buffers start zeroed)");
    tv_dot_kernel<true><<<nblocks, 256, 0, st>>>(a, b, count, partial, out, ticket, pb, rank, world, (unsigned)seq);
    return after_launch("tv_dot_kernel");
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
