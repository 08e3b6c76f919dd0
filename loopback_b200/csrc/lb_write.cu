// Update write with cached key scale and cached scores (sm_100a), plus the small per-update kernels.
//
//   V[s, t, :]     = round_to_storage(h[t, :] - x[t, :])
//   R[s, t]        = rsqrt(mean(V[s, t, :]^2) + eps)            from the ROUNDED update, fp32
//   DOTS[j, s, t]  = q_j . V[s, t, :]   for the queries j >= max(s - 1, 0), i.e. exactly the reads that see update s
//
// Replaces the reference's stacked write kernel (fused_dattn.py:561-585; it scores all queries on tensor cores
// in three-pass TF32). Here the skinny product runs on the CUDA cores in fp32. A CTA takes a tile of 32 or 64 tokens
// and walks the row in 128-byte chunks: phase A is coalesced (8 lanes per token: 128-bit loads of h and x, the rounded
// update stored to V and kept as fp32 in shared memory, the next chunk's loads already in flight), phase B turns the
// tile around -- lanes over tokens, warps over query groups -- so that every lane accumulates complete dot products
// (packed fma.rn.f32x2, query values broadcast from shared memory) and no cross-lane reduction is needed. DOTS is
// token-contiguous ([query][update][token]): a warp stores 32 consecutive floats per query.
#include "lb_common.cuh"
#include "lb_kernels.h"

namespace lb {

// Tile of the write kernel: 32 * TT tokens x all columns, walked in chunks of 128 bytes per token
// (64 bf16 / 32 fp32 columns). 4 warps per CTA; warp w scores queries [w * QPT, (w + 1) * QPT) of the queries that
// will read this update, lane l owns tokens l (and l + 32 when TT == 2) of the tile.
constexpr int kWrThreads = 128;
constexpr int kWrChunkBytes = 128;

template <typename T, int TT, int QPT>
__global__ void __launch_bounds__(kWrThreads, QPT > 12 ? 1 : (TT == 1 ? 8 : 4)) write_kernel(WriteParams p) {
    using S = Store<T>;
    constexpr int VEC = S::kVec;
    constexpr int KC = kWrChunkBytes / S::kBytes;         // columns per chunk
    constexpr int FPT = KC / VEC;                         // 16-byte fragments per token and chunk (8)
    constexpr int TB = 32 * TT;                           // tokens per tile
    constexpr int FRG = TB * FPT / kWrThreads;            // fragments per thread and chunk (2 * TT)
    constexpr int VS = KC + 4;                            // padded row of the fp32 update tile (conflict-free LDS.128)
    constexpr int NQP = 4 * QPT;                          // query rows held per chunk (zero rows past nq)
    constexpr int QF4 = (NQP * KC / 4 + kWrThreads - 1) / kWrThreads;   // float4 of the query chunk per thread
    static_assert(FRG * kWrThreads == TB * FPT, "tile shape");

    extern __shared__ float4 wr_smem4[];
    float *vs = reinterpret_cast<float *>(wr_smem4);                  // [2][TB][VS]
    float *qs = vs + 2 * TB * VS;                                     // [2][NQP][KC]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int d = p.d, nq = p.nq;
    const long long tok0 = (long long)blockIdx.x * TB;
    const T *h = static_cast<const T *>(p.h);
    const T *x = static_cast<const T *>(p.x);
    T *vout = static_cast<T *>(p.v);
    const int nchunks = (d + KC - 1) / KC;
    const bool scores = p.Q != nullptr && nq > 0;

    // phase A fragments of this thread: token (tid >> 3) + 16 m, fragment tid & 7 of the chunk
    const int fr = tid & (FPT - 1);
    uint4 hraw[FRG], xraw[FRG];
    auto fetch = [&](int c) {
        const int col = c * KC + fr * VEC;
#pragma unroll
        for (int m = 0; m < FRG; ++m) {
            const long long tok = min(tok0 + (tid >> 3) + 16 * m, p.n_tok - 1);
            if (col < d) {
                hraw[m] = ld_global_stream_v4(h + tok * d + col);
                xraw[m] = ld_global_stream_v4(x + tok * d + col);
            } else {
                hraw[m] = make_uint4(0, 0, 0, 0);
                xraw[m] = make_uint4(0, 0, 0, 0);
            }
        }
    };

    float2 acc[TT][QPT];
    float2 ss[TT];
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        ss[t] = make_float2(0.f, 0.f);
#pragma unroll
        for (int jj = 0; jj < QPT; ++jj) acc[t][jj] = make_float2(0.f, 0.f);
    }

    fetch(0);
    for (int c = 0; c < nchunks; ++c) {
        const int buf = c & 1;
        float *vb = vs + buf * TB * VS;
        float *qb = qs + buf * NQP * KC;
        // ---- phase A: the update of this chunk -> HBM (rounded once) and, as fp32, -> shared memory
        {
            const int col = c * KC + fr * VEC;
#pragma unroll
            for (int m = 0; m < FRG; ++m) {
                const int tl = (tid >> 3) + 16 * m;
                float hf[VEC], xf[VEC], vf[VEC];
                S::unpack(hraw[m], hf);
                S::unpack(xraw[m], xf);
#pragma unroll
                for (int e = 0; e < VEC; ++e) vf[e] = hf[e] - xf[e];
                const uint4 packed = S::pack(vf);
                S::unpack(packed, vf);                                   // the stored (rounded) values
                if (col < d && tok0 + tl < p.n_tok) st_global_v4(vout + (tok0 + tl) * d + col, packed);
#pragma unroll
                for (int e4 = 0; e4 < VEC / 4; ++e4)
                    *reinterpret_cast<float4 *>(vb + tl * VS + fr * VEC + 4 * e4) =
                        make_float4(vf[4 * e4], vf[4 * e4 + 1], vf[4 * e4 + 2], vf[4 * e4 + 3]);
            }
            if (scores) {
#pragma unroll
                for (int m = 0; m < QF4; ++m) {
                    const int idx = tid + kWrThreads * m;
                    const int jj = idx / (KC / 4), k4 = idx - jj * (KC / 4);
                    const int qcol = c * KC + 4 * k4;
                    float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (jj < nq && qcol < d) q4 = __ldg(reinterpret_cast<const float4 *>(p.Q + (long long)(p.j0 + jj) * d + qcol));
                    if (jj < NQP) *reinterpret_cast<float4 *>(qb + jj * KC + 4 * k4) = q4;
                }
            }
        }
        if (c + 1 < nchunks) fetch(c + 1);           // in flight while this chunk is scored
        __syncthreads();
        // ---- phase B: lanes over tokens; every lane holds complete partial dots, no cross-lane reduction
#pragma unroll 4
        for (int k4 = 0; k4 < KC / 4; ++k4) {
            float4 v4[TT];
#pragma unroll
            for (int t = 0; t < TT; ++t) v4[t] = *reinterpret_cast<const float4 *>(vb + (lane + 32 * t) * VS + 4 * k4);
            if (warp == 0) {
#pragma unroll
                for (int t = 0; t < TT; ++t) {
                    ss[t] = __ffma2_rn(make_float2(v4[t].x, v4[t].y), make_float2(v4[t].x, v4[t].y), ss[t]);
                    ss[t] = __ffma2_rn(make_float2(v4[t].z, v4[t].w), make_float2(v4[t].z, v4[t].w), ss[t]);
                }
            }
            if (scores) {
#pragma unroll
                for (int jj = 0; jj < QPT; ++jj) {
                    const float4 q4 = *reinterpret_cast<const float4 *>(qb + (warp * QPT + jj) * KC + 4 * k4);
#pragma unroll
                    for (int t = 0; t < TT; ++t) {
                        acc[t][jj] = __ffma2_rn(make_float2(v4[t].x, v4[t].y), make_float2(q4.x, q4.y), acc[t][jj]);
                        acc[t][jj] = __ffma2_rn(make_float2(v4[t].z, v4[t].w), make_float2(q4.z, q4.w), acc[t][jj]);
                    }
                }
            }
        }
    }
    // ---- results: one key scale per token, one score per (query, token); lanes are consecutive tokens
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        const long long tok = tok0 + lane + 32 * t;
        if (tok >= p.n_tok) continue;
        if (warp == 0 && p.r != nullptr) p.r[tok] = rsqrtf((ss[t].x + ss[t].y) / (float)d + p.eps);
        if (scores) {
#pragma unroll
            for (int jj = 0; jj < QPT; ++jj) {
                const int j = warp * QPT + jj;
                if (j < nq) p.dots_s[(long long)(p.j0 + j) * p.dots_qstride + tok] = acc[t][jj].x + acc[t][jj].y;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// The same write for a handful of tokens (decode-style batches): gridDim.y CTAs per token, threads over the row, so
// that even 64 tokens occupy most SMs and the query block streams from L2 through all of them. Queries are taken 32 at
// a time (group jg of a token goes to CTA jg mod gridDim.y; CTA 0 of the token also stores the update and its key
// scale): every thread keeps 32 partial dot products, a transposing shuffle reduction leaves query l's warp sum in
// lane l, and the warps' sums meet in shared memory.
// ---------------------------------------------------------------------------------------------------------
constexpr int kWrSmallThreads = 256;
constexpr int kWrSmallFrags = 4;          // fragments per thread: rows up to 256 * 4 * 16 bytes = 16 KiB

__device__ __forceinline__ float transpose_reduce32(float (&vals)[32], int lane) {
    // sum of vals[l] over all lanes, delivered to lane l (31 shuffles for 32 values)
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
__global__ void __launch_bounds__(kWrSmallThreads) write_small_kernel(WriteParams p) {
    using S = Store<T>;
    constexpr int VEC = S::kVec;
    __shared__ float red[kWrSmallThreads / 32][kMaxSources];
    __shared__ float ssred[kWrSmallThreads / 32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long tok = blockIdx.x;
    const int d = p.d, nq = p.Q != nullptr ? p.nq : 0;
    const T *h = static_cast<const T *>(p.h) + tok * d;
    const T *x = static_cast<const T *>(p.x) + tok * d;
    T *vout = static_cast<T *>(p.v) + tok * d;
    float vf[kWrSmallFrags][VEC];
    float ss = 0.f;
#pragma unroll
    for (int m = 0; m < kWrSmallFrags; ++m) {
        const int col = (tid + kWrSmallThreads * m) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) vf[m][e] = 0.f;
        if (col < d) {
            float hf[VEC], xf[VEC];
            S::unpack(ld_global_stream_v4(h + col), hf);
            S::unpack(ld_global_stream_v4(x + col), xf);
#pragma unroll
            for (int e = 0; e < VEC; ++e) vf[m][e] = hf[e] - xf[e];
            const uint4 packed = S::pack(vf[m]);
            S::unpack(packed, vf[m]);                                    // the stored (rounded) values
            if (blockIdx.y == 0) st_global_v4(vout + col, packed);
#pragma unroll
            for (int e = 0; e < VEC; ++e) ss = fmaf(vf[m][e], vf[m][e], ss);
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) ssred[warp] = ss;
    for (int jg = 32 * blockIdx.y; jg < nq; jg += 32 * gridDim.y) {
        float part[32];
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
            part[jj] = 0.f;
            const int j = jg + jj;
            if (j < nq) {
                const float *qrow = p.Q + (long long)(p.j0 + j) * d;
#pragma unroll
                for (int m = 0; m < kWrSmallFrags; ++m) {
                    const int col = (tid + kWrSmallThreads * m) * VEC;
                    if (col < d) {
#pragma unroll
                        for (int e4 = 0; e4 < VEC / 4; ++e4) {
                            const float4 q4 = __ldg(reinterpret_cast<const float4 *>(qrow + col) + e4);
                            part[jj] = fmaf(vf[m][4 * e4], q4.x, part[jj]);
                            part[jj] = fmaf(vf[m][4 * e4 + 1], q4.y, part[jj]);
                            part[jj] = fmaf(vf[m][4 * e4 + 2], q4.z, part[jj]);
                            part[jj] = fmaf(vf[m][4 * e4 + 3], q4.w, part[jj]);
                        }
                    }
                }
            }
        }
        const float tot = transpose_reduce32(part, lane);       // lane l: this warp's sum for query jg + l
        if (jg + lane < nq) red[warp][jg + lane] = tot;
    }
    __syncthreads();
    if (tid == 0 && p.r != nullptr && blockIdx.y == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kWrSmallThreads / 32; ++w) t += ssred[w];
        p.r[tok] = rsqrtf(t / (float)d + p.eps);
    }
    for (int j = tid; j < nq; j += kWrSmallThreads) {
        if ((j >> 5) % (int)gridDim.y != (int)blockIdx.y) continue;
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kWrSmallThreads / 32; ++w) t += red[w][j];
        p.dots_s[(long long)(p.j0 + j) * p.dots_qstride + tok] = t;
    }
}

template <typename T, int TT, int QPT>
static cudaError_t launch_write_t(const WriteParams &p, cudaStream_t stream) {
    constexpr int KC = kWrChunkBytes / Store<T>::kBytes;
    const size_t smem = sizeof(float) * (2 * 32 * TT * (KC + 4) + 2 * 4 * QPT * KC);
    cudaError_t e = cudaFuncSetAttribute(write_kernel<T, TT, QPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const long long tiles = (p.n_tok + 32 * TT - 1) / (32 * TT);
    write_kernel<T, TT, QPT><<<(unsigned)tiles, kWrThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_write_d(const WriteParams &p, int tt, cudaStream_t stream) {
    const int qpt = p.Q && p.nq > 0 ? (p.nq + 3) / 4 : 0;
#define LB_WR(Q_) return tt == 2 ? launch_write_t<T, 2, Q_>(p, stream) : launch_write_t<T, 1, Q_>(p, stream)
    if (qpt <= 2) LB_WR(2);
    if (qpt <= 4) LB_WR(4);
    if (qpt <= 6) LB_WR(6);
    if (qpt <= 12) LB_WR(12);
    if (qpt <= 20) LB_WR(20);
    LB_WR(32);
#undef LB_WR
}

cudaError_t launch_write(int dtype, const WriteParams &p, int sms, cudaStream_t stream) {
    if (p.n_tok == 0) return cudaSuccess;
    if (p.nq > 128) return cudaErrorInvalidValue;
    const int row_frags = p.d / (dtype == LB_DTYPE_BF16 ? 8 : 4);
    if (p.write_tt == 0 && p.n_tok <= 4LL * sms && row_frags <= kWrSmallThreads * kWrSmallFrags) {
        // a decode-sized batch: tiles of 32 tokens would leave most SMs idle
        // one CTA per (token, group of 32 queries) while that stays within a few waves of small CTAs
        int qgroups = (p.nq + 31) / 32, qsplit = qgroups;
        while (qsplit > 1 && p.n_tok * qsplit > 4LL * sms) --qsplit;
        if (qsplit < 1) qsplit = 1;
        const dim3 grid((unsigned)p.n_tok, (unsigned)qsplit);
        if (dtype == LB_DTYPE_BF16) write_small_kernel<__nv_bfloat16><<<grid, kWrSmallThreads, 0, stream>>>(p);
        else write_small_kernel<float><<<grid, kWrSmallThreads, 0, stream>>>(p);
        return cudaGetLastError();
    }
    // two tokens per lane halve the shared-memory traffic per score; one token per lane gives twice the CTAs
    // (better balance when the tiles do not fill the SMs several times over)
    const int tt = p.write_tt ? p.write_tt : (p.n_tok >= (long long)sms * 64 * 3 ? 2 : 1);
    return dtype == LB_DTYPE_BF16 ? launch_write_d<__nv_bfloat16>(p, tt, stream) : launch_write_d<float>(p, tt, stream);
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

// acc = round(beta g), or acc = round(acc + round(beta g)): the boundary blend's gradient of the loop input, in the
// storage type's arithmetic (what autograd's mul and in-place accumulation give).
template <typename T>
__global__ void __launch_bounds__(256) scale_acc_kernel(const T *__restrict__ g, T *__restrict__ acc, float beta, int accumulate,
                                                        long long n_frag) {
    using S = Store<T>;
    constexpr int P = S::kPairs;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const float2 b2 = make_float2(beta, beta);
    for (long long f = (long long)blockIdx.x * blockDim.x + threadIdx.x; f < n_frag; f += stride) {
        float2 v[P];
        S::unpack2(ld_global_stream_v4(g + f * S::kVec), v);
#pragma unroll
        for (int e = 0; e < P; ++e) v[e] = __fmul2_rn(b2, v[e]);
        const uint4 r = accumulate ? S::accum(*reinterpret_cast<const uint4 *>(acc + f * S::kVec), v) : S::pack2v(v);
        st_global_v4(acc + f * S::kVec, r);
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

cudaError_t launch_scale_acc(int dtype, const void *g, void *acc, float beta, int accumulate, long long n_elem, int sms,
                             cudaStream_t stream) {
    if (n_elem == 0) return cudaSuccess;
    const int vec = dtype == LB_DTYPE_BF16 ? 8 : 4;
    const long long n_frag = n_elem / vec;
    const int grid = grid_for(n_frag, 256, sms, 16);
    if (dtype == LB_DTYPE_BF16)
        scale_acc_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(g),
                                                                  static_cast<__nv_bfloat16 *>(acc), beta, accumulate, n_frag);
    else
        scale_acc_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float *>(g), static_cast<float *>(acc), beta,
                                                          accumulate, n_frag);
    return cudaGetLastError();
}

}  // namespace lb
