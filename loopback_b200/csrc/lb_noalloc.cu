// lb_read_bwd_noalloc: the backward read for callers that cannot allocate device memory.
//
// Some hosts of this library hand it buffers but may not call cudaMalloc themselves, nor let a library do so on
// their behalf: an inference or training runtime that pre-plans all device memory at start-up and forbids
// allocation afterwards, a plugin sandbox that exposes only the tensors of the current call, or code running inside
// a region where the allocator is locked. lb_read_bwd needs a few megabytes of scratch for the per-CTA partial rows
// of the query gradient, which such a caller has nowhere to get from. This variant keeps that scratch in a
// file-scope device array of fixed size instead, so the caller passes inputs and outputs only.
//
// Cost and limits, all deliberate:
//   * the array (LB_NOALLOC_MAX_D columns x the library's maximum grid rows, about 3.6 MiB) is part of the loaded
//     module: every GPU on which this library is used holds it until the process exits;
//   * widths above LB_NOALLOC_MAX_D are refused with LB_ERR_UNSUPPORTED (use lb_read_bwd with caller scratch);
//   * all calls on a device share the one array. A call overwrites every row it later reads, so nothing has to be
//     cleared between calls, but two calls that overlap in time on the GPU (different streams, or different
//     threads) race on it and produce a wrong dq. Serialise them on one stream.
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress, which may
//     initialise the module); make that first call outside any stream capture.
#include <mutex>

#include <cuda_runtime.h>

#include "../../include/loopback_b200.h"

extern "C" int lb_fail_message(int code, const char *msg);     // lb_api.cu; internal to the library

namespace {

constexpr int kRows = 304;     // rows lb_read_bwd may use (lb_read_bwd_scratch_bytes(d) / (4 d))

// In host code this name is only a handle for the runtime's symbol functions, never a usable pointer: the device
// address is obtained below, once per device, and that address is what the kernels are given.
static __device__ __align__(256) float g_noalloc_scratch[(size_t)kRows * LB_NOALLOC_MAX_D];

std::mutex g_mu;
float *g_dev_ptr[64] = {};

}  // namespace

#pragma GCC visibility push(default)
extern "C" int lb_read_bwd_noalloc(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g,
                                   const float *gt, const float *cbar, const float *c0, const float *LG,
                                   const float *LSE, const float *LSE0, float *dcbar, float *dq, int64_t n_tok, int d,
                                   int N, int n, int accum, int dtype, void *stream) {
    if (d > LB_NOALLOC_MAX_D || lb_read_bwd_scratch_bytes(d) > sizeof(float) * (size_t)kRows * LB_NOALLOC_MAX_D)
        return lb_fail_message(LB_ERR_UNSUPPORTED,
                               "lb_read_bwd_noalloc: d exceeds LB_NOALLOC_MAX_D, the width its built-in scratch is "
                               "sized for; call lb_read_bwd with caller-provided scratch instead");
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return lb_fail_message(LB_ERR_CUDA, cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return lb_fail_message(LB_ERR_CUDA, "lb_read_bwd_noalloc: device ordinal out of range");
    float *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (g_dev_ptr[dev] == nullptr) {     // set-up, once per device, with that device current
            void *p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess) return lb_fail_message(LB_ERR_CUDA, cudaGetErrorString(e));
            g_dev_ptr[dev] = static_cast<float *>(p);
        }
        scratch = g_dev_ptr[dev];
    }
    return lb_read_bwd(V, R, dV, dR, q, g, gt, cbar, c0, LG, LSE, LSE0, dcbar, dq, scratch, n_tok, d, N, n, accum, dtype,
                       stream);
}
#pragma GCC visibility pop
