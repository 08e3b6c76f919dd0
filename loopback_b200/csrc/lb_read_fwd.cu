// Forward read from stored scores (sm_100a).
//
//   out[t, :] = base[t, :] + sum_{i<n} (tc[t,i] - cbar[t,i]) * V[i, t, :]
//   tc[t,i]   = c0_i + mass * (softmax_i(dots[i,t] r[i,t] / sqrt(d) + lc_i) - softmax_i(lc_i))
//
// Replaces the reference's stored-score read kernel (fused_dattn.py:588-625) and the host preparation around it
// (fused_dattn.py:735-745: log-prior and mass are formed in the kernel from c0).
//
// One persistent CTA per SM walks tiles of BT = NCW / WPT tokens x FR * WPT chunks (a chunk is 512 B of a row;
// NCW = 8, 12 or 16 consumer warps, WPT of them share a token). Normally a tile spans the whole row; only when there
// are too few tokens to fill the GPU is the row also cut into column groups. Warp roles:
//   NCW consumers  warp w owns FR chunks of token w / WPT; lane l owns fragment l of each chunk; fp32 accumulators
//                  held as pairs (fma.rn.f32x2)
//   1 producer     one lane issues TMA tile loads (base tile, then V[0..n) tiles) into a ring of stages
//   4 scalar warps per tile, the n-source softmaxes of its tokens -> coefficient table in shared memory (double
//                  buffered, one tile ahead of the consumers), and the saved TC / LG / LSE / LSE0
// Every wait is bounded (see lb_common.cuh); nothing here spins forever or traps.
#include <cstddef>

#include "lb_common.cuh"
#include "lb_kernels.h"

namespace lb {

constexpr int kFwdScalarWarps = 4;
constexpr int kFwdMaxStages = 32;
constexpr int kFwdMaxBT = 16;                     // tokens per tile == consumer warps (8 or 16)

struct FwdSmemTail {
    float wtab[2][kMaxSources * kFwdMaxBT];       // coefficient deltas w[i][t], double buffered by tile
    float c0[kMaxSources];
    float lc[kMaxSources];
    float mass;
    int abort_flag;
    uint64_t full[kFwdMaxStages];
    uint64_t empty[kFwdMaxStages];
    uint64_t sfull[2];
    uint64_t sempty[2];
};

size_t read_fwd_smem_bytes(int fr, int ncw, int stages, int sps) {
    return 1024 + (size_t)stages * (size_t)sps * (size_t)fr * ncw * kChunkBytes + sizeof(FwdSmemTail);
}

template <typename T, int FR, int NCW>
__global__ void __launch_bounds__((NCW + 1 + kFwdScalarWarps) * 32, 1)
read_fwd_kernel(const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmBase,
                const __grid_constant__ CUtensorMap tmH0, ReadFwdParams p) {
    using S = Store<T>;
    constexpr int VEC = S::kVec;
    constexpr int P = S::kPairs;
    constexpr int BW = kChunkBytes / S::kBytes;               // columns per chunk
    constexpr uint32_t kStageBytes = FR * NCW * kChunkBytes;   // BT tokens x (FR * WPT) chunks
    const int WPT = p.wpt;                                     // consumer warps per token
    const int BT = NCW / WPT;                                  // tokens per tile
    const int CPT = FR * WPT;                                  // chunks per tile (one column group)

    // shared-window addresses of the regions of the dynamic shared memory
    extern __shared__ uint8_t smem_raw[];
    const uint32_t stages_a = (smem_u32(smem_raw) + 1023u) & ~1023u;
    // a stage holds the tile of SPS consecutive sources (one TMA box): small tiles pay the per-stage hand-shake once
    // for up to 4 sources; the base tile takes a stage of its own and uses its first kStageBytes
    const int SPS = p.sps;
    const uint32_t kPitch = (uint32_t)SPS * kStageBytes;
    const uint32_t tail_a = stages_a + (uint32_t)p.stages * kPitch;
    const uint32_t wtab_a = tail_a + offsetof(FwdSmemTail, wtab);
    const uint32_t c0_a = tail_a + offsetof(FwdSmemTail, c0), lc_a = tail_a + offsetof(FwdSmemTail, lc);
    const uint32_t mass_a = tail_a + offsetof(FwdSmemTail, mass), abort_a = tail_a + offsetof(FwdSmemTail, abort_flag);
    const uint32_t full_a = tail_a + offsetof(FwdSmemTail, full), empty_a = tail_a + offsetof(FwdSmemTail, empty);
    const uint32_t sfull_a = tail_a + offsetof(FwdSmemTail, sfull), sempty_a = tail_a + offsetof(FwdSmemTail, sempty);
    constexpr uint32_t kWtabBytes = kMaxSources * kFwdMaxBT * 4;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NS = p.stages;
    const int n = p.n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full_a + 8u * s, 1); mbar_init(empty_a + 8u * s, NCW); }
        for (int b = 0; b < 2; ++b) { mbar_init(sfull_a + 8u * b, kFwdScalarWarps); mbar_init(sempty_a + 8u * b, NCW); }
        sts_s32(abort_a, 0);
        fence_mbar_init();
    }
    if (warp == NCW + 1) {           // prior tables: c0, log-prior, mass
        float m = 0.f;
        for (int i = lane; i < kMaxSources; i += 32) {
            float c = i < n ? p.c0[i] : 0.f;
            if (i < n) { sts_f32(c0_a + 4u * i, c); sts_f32(lc_a + 4u * i, logf(fmaxf(c, 1e-8f))); }
            m += c;
        }
        m = group_sum(m, 32);
        if (lane == 0) sts_f32(mass_a, m);
    }
    __syncthreads();
    const WaitCtx wc{abort_a, p.err_word, p.wait_cycles};

    const int cg_count = p.col_groups;
    const long long n_tiles = (long long)p.tok_tiles * cg_count;

    if (warp < NCW) {
        // ------------------------------------------------------------------ consumers
        int st = 0; uint32_t ph = 0;      // ring position: stage index and its phase parity
        int tcount = 0;
        bool alive = true;      // turned off by a wait that ran out: the warp then finishes its loops without waiting or storing
        const int t = warp / WPT, part = warp - t * WPT;       // this warp's token of the tile and slice of its row
        uint32_t foff[FR];      // byte offset of this lane's fragment k inside a stage (token-major if one 4-D box fills it)
#pragma unroll
        for (int k = 0; k < FR; ++k)
            foff[k] = (uint32_t)((p.rank4 ? t * CPT + part * FR + k : (part * FR + k) * BT + t) * 32 + lane) * 16u;
        long long tt = blockIdx.x / cg_count;
        int cg = (int)(blockIdx.x - tt * cg_count);
        const long long tt_step = gridDim.x / cg_count;
        const int cg_step = (int)(gridDim.x - tt_step * cg_count);
        for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tcount) {
            const long long tok = tt * BT + t;
            const int chunk0 = cg * CPT + part * FR;
            const uint32_t buf = tcount & 1;
            float2 acc[FR][P];
            {   // item 0: the base tile
                if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                const uint32_t sb = stages_a + (uint32_t)st * kPitch;
#pragma unroll
                for (int k = 0; k < FR; ++k) S::unpack2(lds_v4(sb + foff[k]), acc[k]);
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_a + 8u * st);
                if (++st == NS) { st = 0; ph ^= 1u; }
            }
            if (p.blend) {
                // end of an iteration: base = proposal + beta (h0 - proposal), evaluated step by step with the
                // storage type's rounding after each operation, i.e. what the caller's own tensor arithmetic gives
                // (looped_transformer.py:381)
                if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                const uint32_t sb = stages_a + (uint32_t)st * kPitch;
                const float beta = p.beta;
#pragma unroll
                for (int k = 0; k < FR; ++k) {
                    float2 h2[P];
                    S::unpack2(lds_v4(sb + foff[k]), h2);
#pragma unroll
                    for (int e = 0; e < P; ++e) {
                        const float tx = S::round(__fmul_rn(beta, S::round(__fsub_rn(h2[e].x, acc[k][e].x))));
                        const float ty = S::round(__fmul_rn(beta, S::round(__fsub_rn(h2[e].y, acc[k][e].y))));
                        acc[k][e].x = S::round(__fadd_rn(acc[k][e].x, tx));
                        acc[k][e].y = S::round(__fadd_rn(acc[k][e].y, ty));
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_a + 8u * st);
                if (++st == NS) { st = 0; ph ^= 1u; }
            }
            if (alive && !mbar_wait(sfull_a + 8u * buf, (uint32_t)((tcount >> 1) & 1), wc, kDevWaitScalars)) alive = false;
            uint32_t wa = wtab_a + buf * kWtabBytes + 4u * t;
            if (SPS == 1) {
                for (int i = 0; i < n; ++i, wa += 4u * BT) {
                    if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                    const uint32_t sb = stages_a + (uint32_t)st * kPitch;
                    const float wi = lds_f32(wa);
                    const float2 w2 = make_float2(wi, wi);
                    uint4 u[FR];
#pragma unroll
                    for (int k = 0; k < FR; ++k) u[k] = lds_v4(sb + foff[k]);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_a + 8u * st);
                    if (++st == NS) { st = 0; ph ^= 1u; }
#pragma unroll
                    for (int k = 0; k < FR; ++k) {
                        float2 v[P];
                        S::unpack2(u[k], v);
#pragma unroll
                        for (int e = 0; e < P; ++e) acc[k][e] = __ffma2_rn(w2, v[e], acc[k][e]);
                    }
                }
            } else {
                for (int i = 0; i < n; i += SPS) {
                    if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                    uint32_t sb = stages_a + (uint32_t)st * kPitch;
                    const int m = min(SPS, n - i);               // sources past n in the box are never read
                    for (int j = 0; j < m; ++j, wa += 4u * BT, sb += kStageBytes) {
                        const float wi = lds_f32(wa);
                        const float2 w2 = make_float2(wi, wi);
#pragma unroll
                        for (int k = 0; k < FR; ++k) {
                            float2 v[P];
                            S::unpack2(lds_v4(sb + foff[k]), v);
#pragma unroll
                            for (int e = 0; e < P; ++e) acc[k][e] = __ffma2_rn(w2, v[e], acc[k][e]);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_a + 8u * st);
                    if (++st == NS) { st = 0; ph ^= 1u; }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(sempty_a + 8u * buf);
            if (alive && tok < p.n_tok) {
                T *orow = reinterpret_cast<T *>(p.out) + tok * (long long)p.d;
#pragma unroll
                for (int k = 0; k < FR; ++k) {
                    const int col = (chunk0 + k) * BW + lane * VEC;
                    if (col < p.d) st_global_v4(orow + col, S::pack2v(acc[k]));
                }
            }
            tt += tt_step; cg += cg_step;
            if (cg >= cg_count) { cg -= cg_count; ++tt; }
        }
    } else if (warp == NCW) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            tma_prefetch_desc(&tmV);
            tma_prefetch_desc(&tmBase);
            if (p.blend) tma_prefetch_desc(&tmH0);
            const int first_item = p.blend ? -2 : -1;      // items: [-2: proposal,] -1: base or h0, 0..n-1: sources
            int st = 0; uint32_t ph = 0;
            int issued = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const long long tt = tile / cg_count;
                const int cg = (int)(tile - tt * cg_count);
                const int tok0 = (int)(tt * BT);
                const int chunk0 = cg * CPT;
                const int nch = min(CPT, p.chunks - chunk0);
                for (int item = first_item; item < n; item += (item < 0 ? 1 : SPS)) {
                    if (!mbar_wait(empty_a + 8u * st, ph ^ 1u, wc, kDevWaitEmpty)) {
                        ok = false;
                        break;
                    }
                    const uint32_t sb = stages_a + (uint32_t)st * kPitch, fb = full_a + 8u * st;
                    if (p.test_skip_item != 0 && blockIdx.x == 0 && issued + 1 == p.test_skip_item) {
                        // test hook: this copy is left out, so its consumers' bounded wait runs out and the CTA unwinds
                        ++issued;
                        if (++st == NS) { st = 0; ph ^= 1u; }
                        continue;
                    }
                    if (p.rank4) {          // one box: CPT chunks x BT tokens (x SPS sources); what lies past the row or
                                            // the stack is zero-filled and counts toward the bytes all the same
                        mbar_arrive_expect_tx(fb, item < 0 ? kStageBytes : kPitch);
                        if (item < 0) tma_load_3d(sb, (item == first_item) ? &tmBase : &tmH0, fb, 0, chunk0, tok0);
                        else tma_load_4d(sb, &tmV, fb, 0, chunk0, tok0, item);
                    } else {
                        mbar_arrive_expect_tx(fb, (uint32_t)(nch * BT * kChunkBytes));
                        for (int c = 0; c < nch; ++c) {
                            const uint32_t dst = sb + (uint32_t)(c * BT * kChunkBytes);
                            if (item < 0) tma_load_2d(dst, (item == first_item) ? &tmBase : &tmH0, fb, (chunk0 + c) * BW, tok0);
                            else tma_load_3d(dst, &tmV, fb, (chunk0 + c) * BW, tok0, item);
                        }
                    }
                    ++issued;
                    if (++st == NS) { st = 0; ph ^= 1u; }
                }
            }
            if (!ok || lds_volatile_s32(abort_a) != 0) {
                // unwinding (this lane's own wait ran out, or a consumer's did and the consumers stopped waiting for
                // their tiles): let the copies already issued land before the CTA's shared memory is released --
                // the last min(issued, NS) fills, walking the ring backwards from the current position
                long long t0 = clock64();
                int ds = st; uint32_t dp = ph;
                for (int k = 0; k < NS && k < issued; ++k) {
                    if (--ds < 0) { ds = NS - 1; dp ^= 1u; }
                    while (!mbar_try_wait(full_a + 8u * ds, dp)) {
                        if (clock64() - t0 > p.wait_cycles) { atomicCAS(p.err_word, 0, kDevWaitDrain); break; }
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ scalar warps
        const int sw = warp - NCW - 1;
        const int G = n >= 32 ? 32 : (n <= 2 ? 2 : (n <= 4 ? 4 : (n <= 8 ? 8 : (n <= 16 ? 16 : 32))));
        const int TPP = 32 / G;
        const int sub = lane / G, ii = lane % G;
        const float inv = p.inv_sqrt_d, mass = lds_f32(mass_a);
        int tcount = 0;
        for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tcount) {
            const long long tt = tile / cg_count;
            const int cg = (int)(tile - tt * cg_count);
            const uint32_t buf = tcount & 1;
            if (!mbar_wait<true>(sempty_a + 8u * buf, (uint32_t)(((tcount >> 1) & 1) ^ 1), wc, kDevWaitScalarSlot))
                return;
            const uint32_t wt = wtab_a + buf * kWtabBytes;
            // This warp's passes over the tile (pass = sw, sw + 4, ...; TPP tokens per pass). All their global loads
            // are issued before any of them is used, so a tile costs one memory round trip, not one per pass.
            constexpr int U = (NCW + kFwdScalarWarps - 1) / kFwdScalarWarps;    // passes per warp when TPP == 1, WPT == 1
            constexpr int NPL = kMaxSources / 32;
            float rr[U][NPL], dd[U][NPL], cb[U][NPL];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = (sw + kFwdScalarWarps * u) * TPP + sub;
                const long long tok_raw = tt * BT + t;
                const long long tok = tok_raw < p.n_tok ? tok_raw : p.n_tok - 1;
#pragma unroll
                for (int k = 0; k < NPL; ++k) {
                    const int i = ii + 32 * k;
                    rr[u][k] = 0.f; dd[u][k] = 0.f; cb[u][k] = 0.f;
                    if (t < BT && i < n && (k == 0 || G == 32)) {
                        rr[u][k] = __ldg(p.R + (long long)i * p.n_tok + tok);
                        dd[u][k] = __ldg(p.dots + (long long)i * p.n_tok + tok);
                        // installed coefficients: given, or formed from the previous read's (append 1, decay by lam)
                        cb[u][k] = p.tc_prev == nullptr ? __ldg(p.cbar + tok * n + i)
                                                        : (i < n - 1 ? p.lam * __ldg(p.tc_prev + tok * (n - 1) + i) : p.lam);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = (sw + kFwdScalarWarps * u) * TPP + sub;
                if ((sw + kFwdScalarWarps * u) * TPP >= BT) continue;          // warp-uniform
                const long long tok_raw = tt * BT + t;
                const bool tok_ok = tok_raw < p.n_tok && t < BT;
                const long long tok = tok_raw < p.n_tok ? tok_raw : p.n_tok - 1;
                float l[NPL], lcv[NPL];
#pragma unroll
                for (int k = 0; k < NPL; ++k) {
                    const int i = ii + 32 * k;
                    const bool act = i < n && (k == 0 || G == 32);
                    l[k] = -INFINITY; lcv[k] = -INFINITY;
                    if (act) {
                        lcv[k] = lds_f32(lc_a + 4u * i);
                        l[k] = dd[u][k] * rr[u][k] * inv + lcv[k];
                    }
                }
                // the scored softmax and the prior-only softmax go through the same instructions on the same
                // lanes: with a zero query (l == lc) they agree bit for bit, so tc == c0 and out == base exactly
                float mx = l[0], mx0 = lcv[0];
#pragma unroll
                for (int k = 1; k < NPL; ++k) { mx = fmaxf(mx, l[k]); mx0 = fmaxf(mx0, lcv[k]); }
                mx = group_max(mx, G); mx0 = group_max(mx0, G);
                float s = 0.f, s0 = 0.f;
#pragma unroll
                for (int k = 0; k < NPL; ++k) {
                    const int i = ii + 32 * k;
                    const bool act = i < n && (k == 0 || G == 32);
                    s += act ? expf(l[k] - mx) : 0.f;
                    s0 += act ? expf(lcv[k] - mx0) : 0.f;
                }
                s = group_sum(s, G); s0 = group_sum(s0, G);
                const float lse = mx + logf(s), lse0 = mx0 + logf(s0);
#pragma unroll
                for (int k = 0; k < NPL; ++k) {
                    const int i = ii + 32 * k;
                    const bool act = i < n && (k == 0 || G == 32) && t < BT;
                    if (act) {
                        const float pi = expf(l[k] - lse), p0 = expf(lcv[k] - lse0);
                        const float tc = lds_f32(c0_a + 4u * i) + mass * (pi - p0);
                        sts_f32(wt + 4u * (uint32_t)(i * BT + t), tc - cb[u][k]);
                        if (cg == 0 && tok_ok) {
                            p.TC[tok * n + i] = tc;
                            if (p.LG) p.LG[tok * n + i] = l[k];
                        }
                    }
                }
                if (ii == 0 && cg == 0 && tok_ok && p.LSE) { p.LSE[tok] = lse; p.LSE0[tok] = lse0; }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(sfull_a + 8u * buf);
        }
    }
}

template <typename T, int FR, int NCW>
static cudaError_t launch_fwd(const CUtensorMap &tmV, const CUtensorMap &tmBase, const CUtensorMap &tmH0,
                              const ReadFwdParams &p, int grid, cudaStream_t stream) {
    size_t smem = read_fwd_smem_bytes(FR, NCW, p.stages, p.sps);
    cudaError_t e = cudaFuncSetAttribute(read_fwd_kernel<T, FR, NCW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    read_fwd_kernel<T, FR, NCW><<<grid, (NCW + 1 + kFwdScalarWarps) * 32, smem, stream>>>(tmV, tmBase, tmH0, p);
    return cudaGetLastError();
}

cudaError_t launch_read_fwd(int dtype, int fr, int ncw, const CUtensorMap &tmV, const CUtensorMap &tmBase,
                            const CUtensorMap &tmH0, const ReadFwdParams &p, int grid, cudaStream_t stream) {
#define LB_FWD_CASE(TT, F, W) return launch_fwd<TT, F, W>(tmV, tmBase, tmH0, p, grid, stream)
#define LB_FWD_FR(TT, W) \
    switch (fr) { case 1: LB_FWD_CASE(TT, 1, W); case 2: LB_FWD_CASE(TT, 2, W); case 3: LB_FWD_CASE(TT, 3, W); \
                  case 4: LB_FWD_CASE(TT, 4, W); default: break; }
    if (dtype == LB_DTYPE_BF16) {
        if (ncw == 16) { LB_FWD_FR(__nv_bfloat16, 16) } else if (ncw == 12) { LB_FWD_FR(__nv_bfloat16, 12) }
        else if (ncw == 8) { LB_FWD_FR(__nv_bfloat16, 8) }
    } else {
        if (ncw == 16) { LB_FWD_FR(float, 16) } else if (ncw == 12) { LB_FWD_FR(float, 12) }
        else if (ncw == 8) { LB_FWD_FR(float, 8) }
    }
#undef LB_FWD_FR
#undef LB_FWD_CASE
    return cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------------------------------------
// Scores of one query against the first n stored updates, for reads whose scores were not cached by the writes
// (a stack built without queries, or a read issued out of write order): dots[i, t] = q . V[i, t, :].
// Replaces the score half of the reference's online read kernel (fused_dattn.py:426-433).
// One warp per (token, source) row; grid-stride.
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) scores_kernel(const T *__restrict__ V, const float *__restrict__ q,
                                                     float *__restrict__ dots, long long n_tok, int d, int n) {
    using S = Store<T>;
    constexpr int VEC = S::kVec;
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const long long rows = n_tok * n;
    for (long long row = warp0; row < rows; row += nwarps) {     // row = i * n_tok + t
        const T *vp = V + row * d;
        float acc = 0.f;
        for (int c = lane * VEC; c < d; c += 32 * VEC) {
            float v[VEC];
            S::unpack(ld_global_stream_v4(vp + c), v);
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc = fmaf(v[e], __ldg(q + c + e), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) dots[row] = acc;
    }
}

cudaError_t launch_scores(int dtype, const void *V, const float *q, float *dots, long long n_tok, int d, int n,
                          int sms, cudaStream_t stream) {
    long long rows = n_tok * n;
    if (rows == 0) return cudaSuccess;
    long long blocks = (rows + 7) / 8;
    int grid = (int)(blocks < (long long)sms * 8 ? blocks : (long long)sms * 8);
    if (dtype == LB_DTYPE_BF16)
        scores_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(V), q, dots, n_tok, d, n);
    else
        scores_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float *>(V), q, dots, n_tok, d, n);
    return cudaGetLastError();
}

}  // namespace lb
