// One whole forward step for decode-sized batches (sm_100a): the write of update s and the read that follows it, in
// ONE kernel, with the new update kept on chip.
//
//   v = round(h - x) -> V[s];   r = rsqrt(mean(v^2) + eps) -> R[s]
//   l_i = (q . V[i]) R[i] / sqrt(d) + log max(c0_i, 1e-8)   for the n = s + 1 sources (the newest from registers)
//   tc_i = c0_i + mass (softmax_i(l) - softmax_i(log-prior));   out = base + sum_i (tc_i - cbar_i) V[i]
//
// Replaces, for batches too small to fill the GPU with token tiles, the pair of launches the reference makes per step
// (DattnStack.write then the read: _write_stk_kernel + _dattn_fwd_stk_kernel, fused_dattn.py:561-585, :410-456;
// call site modeling_looped_transformer.py:472-481). Like the reference's online read kernel it needs no cached
// scores: two sweeps over the token's stored updates, both served by L2 (the working set of such a step is a few tens
// of MB) -- the first forms every source's score, the second is the weighted sum -- and nothing but V[s], R[s] and the
// outputs is written. The prior-only softmax runs through the same instructions as the scored one, so a zero query
// gives tc == c0 and out == base bit for bit.
//
// One CTA per token. Its threads are SG source groups x CT column threads (thread c of a group owns 16 bytes of the
// row); the groups take the stored sources round-robin in batches of U rows, all loads of a batch in flight at once;
// the groups' partial results are merged at the end. Plain 128-bit loads are used, not TMA.
// (A cluster of two CTAs per token, the sources split between them and the scores and partial rows exchanged through
// distributed shared memory, was built and measured at 64 tokens: the cluster launch and its three barriers cost about
// 4 us per step, more than the second CTA's share of the sweeps saves even at 80 stored updates -- 1.20 ms against
// 0.99 ms for a pass of 80 steps -- so it is not used.)
#include <cstddef>

#include "lb_common.cuh"
#include "lb_kernels.h"

namespace lb {

constexpr int kStepU = 8;                 // rows in flight per thread
constexpr int kStepMaxWarps = 32;

template <typename T>
__device__ __forceinline__ uint4 step_sub(const uint4 &h, const uint4 &x);

template <>
__device__ __forceinline__ uint4 step_sub<__nv_bfloat16>(const uint4 &h, const uint4 &x) {
    auto sub = [](uint32_t a, uint32_t b) {
        const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&a), *reinterpret_cast<const __nv_bfloat162 *>(&b));
        return *reinterpret_cast<const uint32_t *>(&r);
    };
    return make_uint4(sub(h.x, x.x), sub(h.y, x.y), sub(h.z, x.z), sub(h.w, x.w));
}

template <>
__device__ __forceinline__ uint4 step_sub<float>(const uint4 &h, const uint4 &x) {
    return make_uint4(__float_as_uint(__fsub_rn(__uint_as_float(h.x), __uint_as_float(x.x))),
                      __float_as_uint(__fsub_rn(__uint_as_float(h.y), __uint_as_float(x.y))),
                      __float_as_uint(__fsub_rn(__uint_as_float(h.z), __uint_as_float(x.z))),
                      __float_as_uint(__fsub_rn(__uint_as_float(h.w), __uint_as_float(x.w))));
}

// Shared memory: the token's scalar tables, the warps' partial scores [warps per group][source] and the merge buffer
// of the source groups (dynamic, behind this struct).
struct StepSmem {
    float c0[kMaxSources], lc[kMaxSources], w[kMaxSources];      // prior, log-prior, coefficient delta tc - cbar
    float part[kStepMaxWarps][kMaxSources];                       // partial q . V[i] of each warp of the owning group
    float ssq[kStepMaxWarps];                                     // the newest update's squares, per warp of group 0
    float mass;
};

// Two sweeps over the token's stored updates, both from L2: the first forms every source's score (threads over
// columns, each source group takes its sources U rows at a time; one block-wide barrier at the end, none per source),
// one warp then runs both softmaxes over the n scores, and the second sweep is the plain weighted sum the forward read
// makes, with every load independent of every other.
template <typename T, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) step_small_kernel(StepSmallParams p) {
    using S = Store<T>;
    constexpr int VEC = S::kVec;
    constexpr int P = S::kPairs;
    constexpr int U = kStepU;
    extern __shared__ __align__(16) unsigned char smem_dyn[];
    StepSmem &sm = *reinterpret_cast<StepSmem *>(smem_dyn);
    float *merge = reinterpret_cast<float *>(smem_dyn + ((sizeof(StepSmem) + 15) & ~size_t(15)));

    const int CT = p.ct, SG = p.sg;
    const int sg = threadIdx.x / CT, ct = threadIdx.x - sg * CT;
    const int wg = ct >> 5, lane = threadIdx.x & 31, WPG = CT >> 5;       // warp within the group, warps per group
    const long long t = blockIdx.x;
    const int n = p.n, s = n - 1;
    const int col = ct * VEC;
    const bool col_ok = col < p.d;
    const long long row = t * (long long)p.d + col;
    const long long src_stride = p.n_tok * (long long)p.d;
    const T *Vrow = static_cast<const T *>(p.V) + row;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    // the query row, this thread's columns, as pairs
    float2 q2[P];
#pragma unroll
    for (int e4 = 0; e4 < VEC / 4; ++e4) {
        const float4 q4 = col_ok ? __ldg(reinterpret_cast<const float4 *>(p.q + col) + e4) : make_float4(0.f, 0.f, 0.f, 0.f);
        q2[2 * e4] = make_float2(q4.x, q4.y); q2[2 * e4 + 1] = make_float2(q4.z, q4.w);
    }
    // the first warp will run the token's softmaxes: it requests the scalars it needs now, so that their latency
    // passes under the first sweep
    constexpr int NPL = kMaxSources / 32;
    float pre_r[NPL], pre_c0[NPL], pre_cb[NPL];
    if (threadIdx.x < 32) {
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
            const int i = lane + 32 * k;
            pre_r[k] = i < s ? __ldg(p.R + (long long)i * p.n_tok + t) : 0.f;
            pre_c0[k] = i < n ? __ldg(p.c0 + i) : 0.f;
            pre_cb[k] = i < n - 1 ? p.lam * __ldg(p.tc_prev + t * (n - 1) + i) : p.lam;
        }
    }
    auto dot_of = [&](const uint4 &u) {
        float2 v[P];
        S::unpack2(u, v);
        float2 a = make_float2(0.f, 0.f);
#pragma unroll
        for (int e = 0; e < P; ++e) a = __ffma2_rn(q2[e], v[e], a);
        return warp_sum(a.x + a.y);
    };

    // ---- sweep 1: the scores of the stored sources i < s, source i to group i % SG
    for (int i0 = sg; i0 < s; i0 += SG * U) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * SG;
            raw[u] = (i < s && col_ok) ? ld_global_stream_v4(Vrow + i * src_stride) : zero4;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * SG;
            const float dsum = dot_of(raw[u]);
            if (i < s && lane == 0) sm.part[wg][i] = dsum;
        }
    }
    // ---- the write, by group 0: v = round(h - x) -> V[s], its squares and its score; the read's base
    float2 acc[P];
#pragma unroll
    for (int e = 0; e < P; ++e) acc[e] = make_float2(0.f, 0.f);
    uint4 vnew = zero4;
    if (sg == 0) {
        uint4 hv = zero4, xv = zero4;
        if (col_ok) {
            hv = ld_global_stream_v4(static_cast<const T *>(p.h) + row);
            xv = ld_global_stream_v4(static_cast<const T *>(p.x) + row);
        }
        vnew = step_sub<T>(hv, xv);
        if (col_ok) st_global_v4(static_cast<T *>(p.V) + s * src_stride + row, vnew);
        S::unpack2(hv, acc);
        if (p.blend) {
            // end of an iteration: base = h + beta (h0 - h), each operation rounded to the storage type as the caller's
            // own tensor arithmetic rounds it (looped_transformer.py:381)
            float2 h2[P];
            S::unpack2(col_ok ? ld_global_stream_v4(static_cast<const T *>(p.h0) + row) : zero4, h2);
#pragma unroll
            for (int e = 0; e < P; ++e) {
                const float tx = S::round(__fmul_rn(p.beta, S::round(__fsub_rn(h2[e].x, acc[e].x))));
                const float ty = S::round(__fmul_rn(p.beta, S::round(__fsub_rn(h2[e].y, acc[e].y))));
                acc[e].x = S::round(__fadd_rn(acc[e].x, tx));
                acc[e].y = S::round(__fadd_rn(acc[e].y, ty));
            }
        }
        float2 v[P];
        S::unpack2(vnew, v);
        float2 sq = make_float2(0.f, 0.f);
#pragma unroll
        for (int e = 0; e < P; ++e) sq = __ffma2_rn(v[e], v[e], sq);
        const float ssq = warp_sum(sq.x + sq.y), dnew = dot_of(vnew);
        if (lane == 0) { sm.ssq[wg] = ssq; sm.part[wg][s] = dnew; }
    }
    __syncthreads();

    // ---- the n scalars of the token, by the first warp (lanes over sources, four sources per lane): both softmaxes
    // through the same instructions, so a zero query gives tc == c0 exactly and coefficient deltas of exactly zero
    if (threadIdx.x < 32) {
        float ssq = 0.f;
        for (int w = 0; w < WPG; ++w) ssq += sm.ssq[w];
        const float rnew = rsqrtf(ssq / (float)p.d + p.eps);
        if (lane == 0) p.R[(long long)s * p.n_tok + t] = rnew;
        float l[NPL], lcv[NPL], c0v[NPL], mm = 0.f;
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
            const int i = lane + 32 * k;
            l[k] = -INFINITY; lcv[k] = -INFINITY; c0v[k] = 0.f;
            if (i < n) {
                float dsum = 0.f;
                for (int w = 0; w < WPG; ++w) dsum += sm.part[w][i];
                const float r = i < s ? pre_r[k] : rnew;
                c0v[k] = pre_c0[k];
                lcv[k] = logf(fmaxf(c0v[k], 1e-8f));
                l[k] = dsum * r * p.inv_sqrt_d + lcv[k];
            }
            mm += c0v[k];
        }
        const float mass = group_sum(mm, 32);
        float mx = l[0], mx0 = lcv[0];
#pragma unroll
        for (int k = 1; k < NPL; ++k) { mx = fmaxf(mx, l[k]); mx0 = fmaxf(mx0, lcv[k]); }
        mx = group_max(mx, 32); mx0 = group_max(mx0, 32);
        float sum = 0.f, sum0 = 0.f;
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
            const bool act = lane + 32 * k < n;
            sum += act ? expf(l[k] - mx) : 0.f;
            sum0 += act ? expf(lcv[k] - mx0) : 0.f;
        }
        sum = group_sum(sum, 32); sum0 = group_sum(sum0, 32);
        const float lse = mx + logf(sum), lse0 = mx0 + logf(sum0);
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
            const int i = lane + 32 * k;
            if (i < n) {
                const float tc = c0v[k] + mass * (expf(l[k] - lse) - expf(lcv[k] - lse0));
                sm.w[i] = tc - pre_cb[k];
                p.TC[t * n + i] = tc;
                if (p.LG) p.LG[t * n + i] = l[k];
            }
        }
        if (lane == 0 && p.LSE) { p.LSE[t] = lse; p.LSE0[t] = lse0; }
    }
    __syncthreads();

    // ---- sweep 2: out = base + sum_i w_i V[i]; group 0 starts from the base and the newest update (in registers)
    if (sg == 0) {
        float2 v[P];
        S::unpack2(vnew, v);
        const float ws = sm.w[s];
        const float2 w2 = make_float2(ws, ws);
#pragma unroll
        for (int e = 0; e < P; ++e) acc[e] = __ffma2_rn(w2, v[e], acc[e]);
    }
    for (int i0 = sg; i0 < s; i0 += SG * U) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * SG;
            raw[u] = (i < s && col_ok) ? ld_global_stream_v4(Vrow + i * src_stride) : zero4;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * SG;
            const float wi = i < s ? sm.w[i] : 0.f;
            const float2 w2 = make_float2(wi, wi);
            float2 v[P];
            S::unpack2(raw[u], v);
#pragma unroll
            for (int e = 0; e < P; ++e) acc[e] = __ffma2_rn(w2, v[e], acc[e]);
        }
    }
    // ---- merge the source groups into group 0 (fixed order) and store
    if (SG > 1) {
        if (sg > 0) {
            float2 *mb = reinterpret_cast<float2 *>(merge) + ((size_t)(sg - 1) * CT + ct) * P;
#pragma unroll
            for (int e = 0; e < P; ++e) mb[e] = acc[e];
        }
        __syncthreads();
        if (sg == 0) {
            for (int g2 = 1; g2 < SG; ++g2) {
                const float2 *mb = reinterpret_cast<const float2 *>(merge) + ((size_t)(g2 - 1) * CT + ct) * P;
#pragma unroll
                for (int e = 0; e < P; ++e) acc[e] = __fadd2_rn(acc[e], mb[e]);
            }
        }
    }
    if (sg == 0 && col_ok) st_global_v4(static_cast<T *>(p.out) + row, S::pack2v(acc));
}

size_t step_small_smem_bytes(int ct, int sg, int vec) {
    return ((sizeof(StepSmem) + 15) & ~size_t(15)) + (size_t)(sg > 1 ? sg - 1 : 0) * ct * vec * sizeof(float);
}

cudaError_t launch_step_small(int dtype, const StepSmallParams &p, cudaStream_t stream) {
    const int vec = dtype == LB_DTYPE_BF16 ? 8 : 4;
    const size_t smem = step_small_smem_bytes(p.ct, p.sg, vec);
    const int threads = p.ct * p.sg;
#define LB_STEP_LAUNCH(TT, MAXT)                                                                                      \
    {                                                                                                                 \
        cudaError_t e = cudaFuncSetAttribute(step_small_kernel<TT, MAXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             (int)smem);                                                              \
        if (e != cudaSuccess) return e;                                                                               \
        step_small_kernel<TT, MAXT><<<(unsigned)p.n_tok, threads, smem, stream>>>(p);                                 \
        return cudaGetLastError();                                                                                    \
    }
    if (dtype == LB_DTYPE_BF16) {
        if (threads <= 512) LB_STEP_LAUNCH(__nv_bfloat16, 512) else LB_STEP_LAUNCH(__nv_bfloat16, 1024)
    } else {
        if (threads <= 512) LB_STEP_LAUNCH(float, 512) else LB_STEP_LAUNCH(float, 1024)
    }
#undef LB_STEP_LAUNCH
}

}  // namespace lb
