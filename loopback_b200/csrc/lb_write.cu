// Update write with cached key scale and cached scores (sm_100a), plus the small per-update kernels.
//
//   V[s, t, :]     = round_to_storage(h[t, :] - x[t, :])
//   R[s, t]        = rsqrt(mean(V[s, t, :]^2) + eps)            from the ROUNDED update, fp32
//   DOTS[j, s, t]  = q_j . V[s, t, :]   for the queries j >= max(s - 1, 0), i.e. exactly the reads that see update s
//
// Replaces the reference's stacked write kernel (fused_dattn.py:561-585; it scores all queries on tensor cores
// in three-pass TF32). Here the skinny product runs on the CUDA cores in fp32: 128-bit loads, a register tile of
// 4 tokens x 8 queries per warp, and a transposing warp-shuffle reduction. DOTS is token-contiguous
// ([query][update][token]) so that both these stores and the reads' loads are whole sectors.
#include "lb_common.cuh"
#include "lb_kernels.h"

namespace lb {

constexpr int kWrTT = 4;     // tokens per warp pass
constexpr int kWrTQ = 8;     // queries per register tile

// sum of vals[l] over all lanes, delivered to lane l (31 shuffles for 32 values)
__device__ __forceinline__ float transpose_reduce32(float (&vals)[32], int lane) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        const bool up = (lane & s) != 0;
#pragma unroll
        for (int k = 0; k < s; ++k) {
            const float send = up ? vals[k] : vals[k + s];
            const float keep = up ? vals[k + s] : vals[k];
            vals[k] = keep + __shfl_xor_sync(0xffffffffu, send, s);
        }
    }
    return vals[0];
}

template <typename T>
__global__ void __launch_bounds__(256) write_kernel(WriteParams p) {
    using S = Store<T>;
    constexpr int VEC = S::kVec;
    extern __shared__ uint4 wr_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    const int d = p.d;
    const int frags_per_row = d / VEC;                        // 16-byte fragments per token row
    uint4 *vt = wr_smem + (size_t)warp * kWrTT * frags_per_row;   // this warp's [4][d] update tile
    const T *h = static_cast<const T *>(p.h);
    const T *x = static_cast<const T *>(p.x);
    T *vout = static_cast<T *>(p.v);
    const long long groups = (p.n_tok + kWrTT - 1) / kWrTT;

    for (long long grp = (long long)blockIdx.x * warps + warp; grp < groups; grp += (long long)gridDim.x * warps) {
        const long long tok0 = grp * kWrTT;
        float ss[kWrTT] = {0.f, 0.f, 0.f, 0.f};
        // ---- phase A: the update, its store, its sum of squares; the rounded update stays in shared memory
        for (int f = lane; f < frags_per_row; f += 32) {
            uint4 hu[kWrTT], xu[kWrTT];
#pragma unroll
            for (int t = 0; t < kWrTT; ++t) {
                const long long tok = min(tok0 + t, p.n_tok - 1);
                hu[t] = ld_global_stream_v4(h + tok * d + f * VEC);
                xu[t] = ld_global_stream_v4(x + tok * d + f * VEC);
            }
#pragma unroll
            for (int t = 0; t < kWrTT; ++t) {
                float hf[VEC], xf[VEC], vf[VEC];
                S::unpack(hu[t], hf);
                S::unpack(xu[t], xf);
#pragma unroll
                for (int e = 0; e < VEC; ++e) vf[e] = hf[e] - xf[e];
                const uint4 packed = S::pack(vf);
                S::unpack(packed, vf);                                   // the stored (rounded) values
#pragma unroll
                for (int e = 0; e < VEC; ++e) ss[t] = fmaf(vf[e], vf[e], ss[t]);
                vt[t * frags_per_row + f] = packed;
                if (tok0 + t < p.n_tok) st_global_v4(vout + (tok0 + t) * d + f * VEC, packed);
            }
        }
#pragma unroll
        for (int t = 0; t < kWrTT; ++t) ss[t] = warp_sum(ss[t]);
        if (p.r != nullptr && lane < kWrTT && tok0 + lane < p.n_tok) {
            const float mine = lane == 0 ? ss[0] : (lane == 1 ? ss[1] : (lane == 2 ? ss[2] : ss[3]));
            p.r[tok0 + lane] = rsqrtf(mine / (float)d + p.eps);
        }
        if (p.Q == nullptr || p.nq <= 0) continue;
        __syncwarp();
        // ---- phase B: scores of the 4 tokens against the queries that will read this update
        for (int jg = 0; jg < p.nq; jg += kWrTQ) {
            float acc[32];
#pragma unroll
            for (int k = 0; k < 32; ++k) acc[k] = 0.f;
            for (int f = lane; f < frags_per_row; f += 32) {
                float vf[kWrTT][VEC];
#pragma unroll
                for (int t = 0; t < kWrTT; ++t) S::unpack(vt[t * frags_per_row + f], vf[t]);
#pragma unroll
                for (int jj = 0; jj < kWrTQ; ++jj) {
                    const int j = min(jg + jj, p.nq - 1) + p.j0;      // clamped: surplus lanes recompute the last query
                    const float4 *qp = reinterpret_cast<const float4 *>(p.Q + (long long)j * d + f * VEC);
                    float qf[VEC];
#pragma unroll
                    for (int e4 = 0; e4 < VEC / 4; ++e4) {
                        const float4 q4 = __ldg(qp + e4);
                        qf[4 * e4] = q4.x; qf[4 * e4 + 1] = q4.y; qf[4 * e4 + 2] = q4.z; qf[4 * e4 + 3] = q4.w;
                    }
#pragma unroll
                    for (int t = 0; t < kWrTT; ++t)
#pragma unroll
                        for (int e = 0; e < VEC; ++e) acc[t * kWrTQ + jj] = fmaf(vf[t][e], qf[e], acc[t * kWrTQ + jj]);
                }
            }
            const float tot = transpose_reduce32(acc, lane);       // lane = t * 8 + jj
            const int t = lane / kWrTQ, jj = lane % kWrTQ;
            if (jg + jj < p.nq && tok0 + t < p.n_tok)
                p.dots_s[(long long)(p.j0 + jg + jj) * p.dots_qstride + tok0 + t] = tot;
        }
        __syncwarp();
    }
}

cudaError_t launch_write(int dtype, const WriteParams &p, int sms, cudaStream_t stream) {
    if (p.n_tok == 0) return cudaSuccess;
    const int elem = dtype == LB_DTYPE_BF16 ? 2 : 4;
    const size_t per_warp = (size_t)kWrTT * p.d * elem;
    int warps = 8;
    while (warps > 1 && per_warp * warps > 96 * 1024) warps >>= 1;
    const size_t smem = per_warp * warps;
    const long long groups = (p.n_tok + kWrTT - 1) / kWrTT;
    long long blocks = (groups + warps - 1) / warps;
    const long long cap = (long long)sms * 16;
    const int grid = (int)(blocks < cap ? blocks : cap);
    cudaError_t e;
    if (dtype == LB_DTYPE_BF16) {
        e = cudaFuncSetAttribute(write_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        write_kernel<__nv_bfloat16><<<grid, warps * 32, smem, stream>>>(p);
    } else {
        e = cudaFuncSetAttribute(write_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        write_kernel<float><<<grid, warps * 32, smem, stream>>>(p);
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------
// Key scale of a free-standing update (list layout): r[t] = rsqrt(mean(x[t,:]^2) + eps).
// Replaces fused_dattn.py:206-215. One warp per token.
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) rstd_fwd_kernel(const T *__restrict__ x, float *__restrict__ r,
                                                       long long n_tok, int d, float eps) {
    using S = Store<T>;
    constexpr int VEC = S::kVec;
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long tok = warp0; tok < n_tok; tok += nwarps) {
        float ss = 0.f;
        for (int c = lane * VEC; c < d; c += 32 * VEC) {
            float v[VEC];
            S::unpack(ld_global_stream_v4(x + tok * d + c), v);
#pragma unroll
            for (int e = 0; e < VEC; ++e) ss = fmaf(v[e], v[e], ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) r[tok] = rsqrtf(ss / (float)d + eps);
    }
}

// Gradient of the key scale: gx = gr (-r^3 / d) x. mode 0 writes it (fused_dattn.py:218-229); mode 1 adds its
// storage-rounded value into gx and rounds the sum, which is how the reference accumulates it into the update's
// gradient slice (fused_dattn.py:539-552).
template <typename T>
__global__ void __launch_bounds__(256) rstd_bwd_kernel(const T *__restrict__ x, const float *__restrict__ r,
                                                       const float *__restrict__ gr, T *__restrict__ gx,
                                                       long long n_tok, int d, int mode) {
    using S = Store<T>;
    constexpr int VEC = S::kVec;
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long tok = warp0; tok < n_tok; tok += nwarps) {
        const float rr = r[tok];
        const float k = gr[tok] * (-(rr * rr * rr)) / (float)d;
        for (int c = lane * VEC; c < d; c += 32 * VEC) {
            float v[VEC], o[VEC];
            S::unpack(ld_global_stream_v4(x + tok * d + c), v);
            if (mode == 0) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) o[e] = k * v[e];
            } else {
                float prev[VEC];
                S::unpack(*reinterpret_cast<const uint4 *>(gx + tok * d + c), prev);
#pragma unroll
                for (int e = 0; e < VEC; ++e) o[e] = prev[e] + S::round(k * v[e]);
            }
            st_global_v4(gx + tok * d + c, S::pack(o));
        }
    }
}

// out = -g: the gradient the write hands to the block input (fused_dattn.py:693-695).
template <typename T>
__global__ void __launch_bounds__(256) neg_kernel(const T *__restrict__ g, T *__restrict__ out, long long n_frag) {
    using S = Store<T>;
    constexpr int VEC = S::kVec;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long f = (long long)blockIdx.x * blockDim.x + threadIdx.x; f < n_frag; f += stride) {
        float v[VEC];
        S::unpack(ld_global_stream_v4(g + f * VEC), v);
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[e] = -v[e];
        st_global_v4(out + f * VEC, S::pack(v));
    }
}

static int grid_for(long long work_items, int per_block, int sms, int waves) {
    long long blocks = (work_items + per_block - 1) / per_block;
    const long long cap = (long long)sms * waves;
    if (blocks < 1) blocks = 1;
    return (int)(blocks < cap ? blocks : cap);
}

cudaError_t launch_rstd_fwd(int dtype, const void *x, float *r, long long n_tok, int d, float eps, int sms,
                            cudaStream_t stream) {
    if (n_tok == 0) return cudaSuccess;
    const int grid = grid_for(n_tok, 8, sms, 16);
    if (dtype == LB_DTYPE_BF16)
        rstd_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), r, n_tok, d, eps);
    else
        rstd_fwd_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float *>(x), r, n_tok, d, eps);
    return cudaGetLastError();
}

cudaError_t launch_rstd_bwd(int dtype, const void *x, const float *r, const float *gr, void *gx, long long n_tok,
                            int d, int mode, int sms, cudaStream_t stream) {
    if (n_tok == 0) return cudaSuccess;
    const int grid = grid_for(n_tok, 8, sms, 16);
    if (dtype == LB_DTYPE_BF16)
        rstd_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), r, gr,
                                                                 static_cast<__nv_bfloat16 *>(gx), n_tok, d, mode);
    else
        rstd_bwd_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float *>(x), r, gr,
                                                         static_cast<float *>(gx), n_tok, d, mode);
    return cudaGetLastError();
}

cudaError_t launch_neg(int dtype, const void *g, void *out, long long n_elem, int sms, cudaStream_t stream) {
    if (n_elem == 0) return cudaSuccess;
    const int vec = dtype == LB_DTYPE_BF16 ? 8 : 4;
    const long long n_frag = n_elem / vec;
    const int grid = grid_for(n_frag, 256, sms, 16);
    if (dtype == LB_DTYPE_BF16)
        neg_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(g),
                                                            static_cast<__nv_bfloat16 *>(out), n_frag);
    else
        neg_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float *>(g), static_cast<float *>(out), n_frag);
    return cudaGetLastError();
}

}  // namespace lb
