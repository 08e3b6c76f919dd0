// One-shot all-reduce of the query gradient over the GPUs of one node, through peer memory (NVLink / NVSwitch).
//
// Every rank's backward leaves its own (N - 1, d) fp32 query gradient in a buffer its peers can address. One small
// kernel per rank then sums all ranks' buffers, in rank order (every rank gets the same bits), into the rank's result.
// The reference gets this sum from FSDP's reduce-scatter of query.grad (trainer/flame/models/parallelize_fla.py:549-554);
// at 94 KB (config 2) an NCCL all-reduce is all launch and protocol latency, which plain peer loads avoid.
//
// Synchronisation is per CTA and per slice: CTA b of every rank owns the same slice of the buffer and talks only to
// the CTAs b of its peers, through flag words that carry a call counter ("epoch", kept on the device so that a CUDA
// graph replays correctly):
//   1. ready: CTA b stores its epoch into slot (phase 0, own rank, b) of EVERY rank's flag block (st.release.sys), then
//      waits until slot (phase 0, r, b) of its own block has reached the epoch for every r;
//   2. it sums slice b of the W buffers with ld.relaxed.sys loads (no multicast, no TMA) and writes the result;
//   3. done: the same handshake on phase 1, so that when the kernel ends no peer is still reading this rank's
//      buffer and the next pass may overwrite it.
// Every wait is bounded: past the limit the CTA records kDevWaitPeer in the device error word, skips its sum, still
// signals (so that its peers are not held up by it) and returns.
// The kernels of different ranks wait on one another, so each rank must run on a GPU of its own.
#include "lb_common.cuh"
#include "lb_kernels.h"

namespace lb {

namespace {

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_relaxed_sys_f4(const float *p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// thread r < world: tell rank r, then wait for rank r; returns false when the wait ran out
__device__ __forceinline__ bool handshake(const PeerReduceParams &p, int phase, unsigned epoch, int r, int b) {
    st_release_sys(p.flags[r] + ((phase * kMaxPeers + p.rank) * kPeerCtas + b), epoch);
    const unsigned *mine = p.flags[p.rank] + ((phase * kMaxPeers + r) * kPeerCtas + b);
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
        if (clock64() - t0 > p.wait_cycles) {
            atomicCAS(p.err_word, 0, (int)kDevWaitPeer);
            return false;
        }
        __nanosleep(64);
    }
    return true;
}

__global__ void __launch_bounds__(256) peer_allreduce_kernel(const PeerReduceParams p) {
    __shared__ unsigned s_epoch;
    __shared__ int s_ok;
    const int b = blockIdx.x;
    if (threadIdx.x == 0) {
        unsigned *ctr = p.flags[p.rank] + 2 * kMaxPeers * kPeerCtas + b;   // this CTA's call counter
        s_epoch = *ctr + 1u;
        *ctr = s_epoch;
        s_ok = 1;
    }
    __syncthreads();
    const unsigned epoch = s_epoch;
    // the rows were written by earlier kernels of this stream: make them visible at system scope before the flag
    __threadfence_system();
    if ((int)threadIdx.x < p.world && !handshake(p, 0, epoch, threadIdx.x, b)) s_ok = 0;
    __syncthreads();
    if (s_ok) {
        const long long lo = (long long)b * p.slice4, hi = min(lo + p.slice4, p.n4);
        for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            // every rank's group is requested before the first is used: one NVLink round trip per group, not one per rank
            float4 v[kMaxPeers];
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
                if (r < p.world) v[r] = ld_relaxed_sys_f4(p.bufs[r] + 4 * i);
            float4 acc = v[0];
#pragma unroll
            for (int r = 1; r < kMaxPeers; ++r)
                if (r < p.world) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
            reinterpret_cast<float4 *>(p.out)[i] = acc;
        }
    }
    __syncthreads();
    if ((int)threadIdx.x < p.world) handshake(p, 1, epoch, threadIdx.x, b);
}

}  // namespace

int peer_allreduce_ctas(long long n4) {
    long long g = (n4 + 255) / 256;           // one 16-byte group per thread while the CTAs last
    return (int)(g < 1 ? 1 : (g > kPeerCtas ? kPeerCtas : g));
}

cudaError_t launch_peer_allreduce(PeerReduceParams p, cudaStream_t stream) {
    const int grid = peer_allreduce_ctas(p.n4);
    p.slice4 = (p.n4 + grid - 1) / grid;
    peer_allreduce_kernel<<<grid, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace lb
