// Backward of one read over the stacked updates (sm_100a): one kernel, one pass over V, one pass over dV.
//
// Given g = dL/dout [n_tok, d] and gt = dL/dtc [n_tok, n] (optional), with p_i = exp(LG_i - LSE) saved by the forward:
//   phase 1 (streams V[i] once):   gd_i = g . v_i     gp_i = mass (gd_i + gt_i)     S = sum_i p_i gp_i
//                                  A = sum_i p_i r_i gp_i v_i      B = sum_i p_i r_i v_i
//                                  dq partial += A - S B                       (scaled by 1/sqrt(d) at the end)
//   scalars:                       dz_i = p_i (gp_i - S)    dR[i] (+)= dz_i (LG_i - lc_i) / r_i    dcbar_i = -gd_i
//   phase 2 (streams dV[i] once):  dV[i] (+)= w_i g + dz_i r_i q / sqrt(d),   w_i = c0_i - cbar_i + mass (p_i - p0_i)
// In accumulate mode the old dV / dR are read and the sum is rounded to the storage type after the new term was
// rounded on its own (bf16: exactly what a bf16 autograd add_ of a bf16 gradient does).
//
// Replaces the reference's two backward kernels and the torch reduction between them (fused_dattn.py:459-536,
// :761-793): no GD / SACC round trip through HBM, g is read once, and the query gradient leaves the kernel as one
// partial row per CTA.
//
// Tiles are BT = NCW / WPT tokens x the full row; a token's row is split over WPT consumer warps (FR chunks of
// 512 B each). Warp roles: NCW consumer warps, 1 TMA producer lane, 2 scalar warps that prepare the
// per-(token, source) tables of the next tile. The element math runs on pairs (fma.rn.f32x2). All waits are bounded.
#pragma once

#include <cstddef>
#include <type_traits>

#include "lb_common.cuh"
#include "lb_kernels.h"

#ifndef LB_BWD_UNROLL
#define LB_BWD_UNROLL 4
#endif


namespace lb {

// scalar warps per CTA: 2, or 1 in the half-size CTA (4 consumer warps) of which two share an SM
constexpr int bwd_scalar_warps(int ncw) { return ncw == 4 ? 1 : 2; }
constexpr int bwd_ctas_per_sm(int ncw) { return ncw == 4 ? 2 : 1; }
constexpr int kBwdMaxStages = 12;
constexpr int kBwdTables = 6;     // P, R, GT, W, ZL, DRP
constexpr int kBwdMaxNcw = 16;

struct BwdSmemTail {
    float c0[kMaxSources];
    float lc[kMaxSources];
    float mass;
    int abort_flag;
    alignas(16) float xch[2][kBwdMaxNcw][4];    // partial g.v of the token's warps (up to 4 sources at a time, read and
                                                // written as 16-byte vectors), double buffered
    float fin[kBwdMaxNcw];                      // per token: coefficient of the key-scale term of the finalised source
    float fin0[kBwdMaxNcw];                     // ... and of update 0, which the step-1 backward finishes as well
    uint64_t full[kBwdMaxStages];
    uint64_t empty[kBwdMaxStages];
    uint64_t sfull[2];
    uint64_t sempty[2];
};

static_assert(offsetof(BwdSmemTail, xch) % 16 == 0, "the exchange buffers are accessed with 16-byte loads and stores");
static_assert(offsetof(BwdSmemTail, full) % 8 == 0, "mbarriers are 8-byte objects");

// dynamic shared memory: [stages][tables 2 x 6 x n_pad*BT][gdkq n_pad*BT][dq slots][q: chunks*512/elem floats][tail]
__host__ __device__ inline int bwd_npad(int n) { return (n + 3) & ~3; }
__host__ __device__ inline size_t bwd_table_floats(int n, int bt) { return (size_t)bwd_npad(n) * bt; }

// (read_bwd_smem_bytes, declared in lb_kernels.h, is defined in lb_read_bwd.cu)

template <typename T, int FR, int NCW, bool SOLO, int MODE>
__global__ void __launch_bounds__((NCW + 1 + bwd_scalar_warps(NCW)) * 32, bwd_ctas_per_sm(NCW))
read_bwd_kernel(const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG,
                const __grid_constant__ CUtensorMap tmDV, const __grid_constant__ CUtensorMap tmH0, ReadBwdParams p) {
    using S = Store<T>;
    constexpr int VEC = S::kVec;
    constexpr int P = S::kPairs;
    constexpr int V4 = VEC / 4;
    constexpr int BW = kChunkBytes / S::kBytes;
    constexpr uint32_t kStageBytes = FR * NCW * kChunkBytes;
    constexpr int kConsumerThreads = NCW * 32;
    constexpr bool STEP = MODE >= 1, DEFER = MODE == 2;
    constexpr int kBwdScalarWarps = bwd_scalar_warps(NCW);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NS = p.stages, n = p.n, WPT = SOLO ? 1 : p.wpt, BT = NCW / WPT;
    const uint32_t tfl4 = (uint32_t)bwd_table_floats(n, BT) * 4u;      // bytes of one table
    const int J = DEFER ? p.n_total - n : 0;                           // backward steps that ran before this one
    const uint32_t ftl4 = (uint32_t)bwd_table_floats(J, BT) * 4u;      // bytes of one table of their scalars

    // shared-window addresses of the regions of the dynamic shared memory
    extern __shared__ uint8_t smem_raw[];
    const uint32_t stages_a = (smem_u32(smem_raw) + 1023u) & ~1023u;
    // a stage: one tile; in the deferred form a g tile travels with the query row of its step right behind it
    const uint32_t pitch = DEFER ? kStageBytes + (uint32_t)p.qrow_bytes : kStageBytes;
    const uint32_t tables_a = stages_a + (uint32_t)NS * pitch;
    const uint32_t gdkq_a = tables_a + 2u * kBwdTables * tfl4;
    const uint32_t ft_a = gdkq_a + tfl4;                               // DEFER: 2 buffers x 4 tables (w, kq; w, kq of update 0)
    const uint32_t slots_a = (ft_a + (DEFER ? 8u * ftl4 : 0u) + 15u) & ~15u;
    const uint32_t qsm_a = slots_a + (uint32_t)(FR * V4 * kConsumerThreads) * 16u;
    const uint32_t tail_a = (qsm_a + (uint32_t)(FR * WPT * 32 * V4) * 16u + 15u) & ~15u;
    const uint32_t c0_a = tail_a + offsetof(BwdSmemTail, c0), lc_a = tail_a + offsetof(BwdSmemTail, lc);
    const uint32_t mass_a = tail_a + offsetof(BwdSmemTail, mass), abort_a = tail_a + offsetof(BwdSmemTail, abort_flag);
    const uint32_t xch_a = tail_a + offsetof(BwdSmemTail, xch), fin_a = tail_a + offsetof(BwdSmemTail, fin);
    const uint32_t fin0_a = tail_a + offsetof(BwdSmemTail, fin0);
    const uint32_t full_a = tail_a + offsetof(BwdSmemTail, full), empty_a = tail_a + offsetof(BwdSmemTail, empty);
    const uint32_t sfull_a = tail_a + offsetof(BwdSmemTail, sfull), sempty_a = tail_a + offsetof(BwdSmemTail, sempty);

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full_a + 8u * s, 1); mbar_init(empty_a + 8u * s, NCW); }
        for (int b = 0; b < 2; ++b) { mbar_init(sfull_a + 8u * b, kBwdScalarWarps); mbar_init(sempty_a + 8u * b, NCW); }
        sts_s32(abort_a, 0);
        fence_mbar_init();
    }
    if (warp == NCW + 1) {
        float m = 0.f;
        for (int i = lane; i < kMaxSources; i += 32) {
            float c = i < n ? p.c0[i] : 0.f;
            if (i < n) { sts_f32(c0_a + 4u * i, c); sts_f32(lc_a + 4u * i, logf(fmaxf(c, 1e-8f))); }
            m += c;
        }
        m = group_sum(m, 32);
        if (lane == 0) sts_f32(mass_a, m);
    }
    if (warp < NCW) {
#pragma unroll
        for (int k = 0; k < FR * V4; ++k)
            sts_f4(slots_a + (uint32_t)(k * kConsumerThreads + threadIdx.x) * 16u, make_float4(0.f, 0.f, 0.f, 0.f));
        // the query stays in shared memory for the whole kernel: no global load sits in the consumers' path
        for (int f4 = threadIdx.x; f4 < FR * WPT * 32 * V4; f4 += kConsumerThreads)
            sts_f4(qsm_a + 16u * f4, f4 * 4 < p.d ? __ldg(reinterpret_cast<const float4 *>(p.q) + f4)
                                                  : make_float4(0.f, 0.f, 0.f, 0.f));
    }
    __syncthreads();
    const WaitCtx wc{abort_a, p.err_word, p.wait_cycles};
    const long long n_tiles = p.tok_tiles;
    // the old h0 gradient comes as one more tile (one-warp-per-token shapes; the others leave h0's gradient to a kernel of its own)
    const bool dh0_rmw = STEP && SOLO && p.dh0 != nullptr && p.dh0_accum != 0;
    const bool fin2 = DEFER && p.fin2 != 0;       // also finish update 0 (the step-1 backward)
    const int items_per_tile = DEFER ? 1 + (dh0_rmw ? 1 : 0) + n + J + (fin2 ? 1 + J : 0)
                                     : 1 + n + (p.accum ? n : 0) + (dh0_rmw ? 1 : 0);
    // stage layout: token-major [t][chunk][512 B] when one 4-D TMA box fills a stage, chunk-major [chunk][t][512 B]
    // when the row is fetched chunk by chunk
    const int tstride = p.rank4 ? p.chunks : 1, cstride = p.rank4 ? 1 : BT;

    if (warp < NCW) {
        // ------------------------------------------------------------------ consumers
        const int t = warp / WPT;                 // token of the tile
        const int part = warp - t * WPT;          // which slice of the row
        const int chunk0 = part * FR;
        const float mass = lds_f32(mass_a), inv = p.inv_sqrt_d;
        const int bar_id = 1 + t, bar_threads = WPT * 32;
        const uint32_t BT4 = 4u * BT, t4 = 4u * t;
        int st = 0; uint32_t ph = 0;              // ring position: stage index and its phase parity
        int tcount = 0;
        // A wait that runs out must not make this warp leave: its sibling warps meet it at named barriers. It
        // turns `alive` off instead, and the warp walks the remaining (finite) loop structure without waiting or
        // storing, so every barrier still gets all its arrivals.
        bool alive = true;
        bool valid[FR];
        uint32_t foff[FR];                        // byte offset of this lane's fragment k inside a stage
#pragma unroll
        for (int k = 0; k < FR; ++k) {
            valid[k] = chunk0 + k < p.chunks;
            foff[k] = (uint32_t)((t * tstride + (chunk0 + k) * cstride) * 32 + lane) * 16u;
        }
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
        for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tcount) {
            const long long tok = tile * BT + t;
            const bool tok_in = tok < p.n_tok;
            const uint32_t buf = tcount & 1;
            // tables of this tile, entry (i, t) of table k at tb + k * tfl4 + i * BT4 + t4:  P, R, GT, W, ZL, DRP
            const uint32_t tb = tables_a + buf * kBwdTables * tfl4 + t4;
            const uint32_t gk = gdkq_a + t4;
            // ---- g tile -> registers (as fp32 pairs)
            // (the one-warp-per-token shapes keep g packed and unpack it where it is used, to leave room for 4 fragments
            // per lane; unpacked it costs the 4-fragment shape 200 bytes of spills. The deferred form uses g once per
            // source only, in the dot product, which takes it packed: every shape keeps it packed there)
            constexpr bool PACKG = SOLO || DEFER;
            float2 g2[PACKG ? 1 : FR][P];
            uint4 gpk[PACKG ? FR : 1];
            auto load_g = [&](int k, float2 (&gf)[P]) {          // g fragment k as fp32 pairs
                if constexpr (PACKG) S::unpack2(gpk[k], gf);
                else {
#pragma unroll
                    for (int e = 0; e < P; ++e) gf[e] = g2[k][e];
                }
            };
            {
                if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                const uint32_t sb = stages_a + (uint32_t)st * pitch;
#pragma unroll
                for (int k = 0; k < FR; ++k) {
                    const uint4 u = valid[k] ? lds_v4(sb + foff[k]) : zero4;
                    if constexpr (PACKG) gpk[k] = u; else S::unpack2(u, g2[k]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_a + 8u * st);
                if (++st == NS) { st = 0; ph ^= 1u; }
            }
            if constexpr (DEFER) {
                // the upstream gradient is kept for the backward steps that follow (autograd frees its own copy)
                T *grow = reinterpret_cast<T *>(p.Gst) + ((long long)(n - 1) * p.n_tok + tok) * (long long)p.d + chunk0 * BW + lane * VEC;
#pragma unroll
                for (int k = 0; k < FR; ++k) {
                    uint4 u;
                    if constexpr (PACKG) u = gpk[k]; else u = S::pack2v(g2[k]);
                    if (alive && tok_in && (chunk0 + k) * BW + lane * VEC < p.d) st_global_v4(grow + k * BW, u);
                }
            }
            if (STEP && SOLO && p.dh0 != nullptr) {
                // the read closed an iteration (base = h + beta (h0 - h)): h0's share of g, round(beta g), leaves at
                // once -- written, or added to what earlier backward reads of the pass left there (that tile is the
                // next item of the ring)
                uint32_t sb0 = 0;
                if (dh0_rmw) {
                    if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                    sb0 = stages_a + (uint32_t)st * pitch;
                }
                const float2 b2 = make_float2(p.beta, p.beta);
#pragma unroll
                for (int k = 0; k < FR; ++k) {
                    float2 bg[P];
                    load_g(k, bg);
#pragma unroll
                    for (int e = 0; e < P; ++e) bg[e] = __fmul2_rn(b2, bg[e]);
                    const uint4 acc0 = dh0_rmw ? S::accum(valid[k] ? lds_v4(sb0 + foff[k]) : zero4, bg) : S::pack2v(bg);
                    const int col = (chunk0 + k) * BW + lane * VEC;
                    if (alive && tok_in && col < p.d)
                        st_global_v4(reinterpret_cast<T *>(p.dh0) + tok * (long long)p.d + col, acc0);
                }
                if (dh0_rmw) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_a + 8u * st);
                    if (++st == NS) { st = 0; ph ^= 1u; }
                }
            }
            if (alive && !mbar_wait(sfull_a + 8u * buf, (uint32_t)((tcount >> 1) & 1), wc, kDevWaitScalars)) alive = false;

            // ---- phase 1: one pass over the sources, software-pipelined two deep: iteration i loads source i and starts
            // the warp reduction of g . v_i; the reduced value is published to the token's other warps one iteration
            // later and consumed (A, B accumulation of that source) two iterations later, so neither the shuffle chain
            // nor the exchange barrier sits on an iteration's critical path
            float2 A[FR][P], B[FR][P];
            uint4 v1[FR], v2[FR];                 // packed fragments of sources i-1 and i-2
#pragma unroll
            for (int k = 0; k < FR; ++k) {
                v1[k] = zero4; v2[k] = zero4;
#pragma unroll
                for (int e = 0; e < P; ++e) { A[k][e] = make_float2(0.f, 0.f); B[k][e] = make_float2(0.f, 0.f); }
            }
            float sacc = 0.f, d1 = 0.f, d2 = 0.f;  // this warp's g . v of sources i-1 and i-2
            constexpr int DEPTH = SOLO ? 1 : 2;
            // One iteration, specialised at compile time on whether it still loads a source (LOAD: i < n) and whether a
            // source is ready to be accumulated (ACC: i >= DEPTH), so that the steady-state body is straight-line code:
            // the accumulation of the older source is independent of the new source's dot product and shuffle
            // reduction, and the five dependent shuffle steps are written between its fragments so that their latency
            // is covered by its FMAs instead of stalling the warp.
            auto iter = [&](int i, auto load_tag, auto acc_tag) {
                constexpr bool LOAD = decltype(load_tag)::value, ACC = decltype(acc_tag)::value;
                if (WPT > 1 && i >= 1 && i <= n && lane == 0) sts_f32(xch_a + 16u * (((i - 1) & 1) * kBwdMaxNcw + warp), d1);
                uint4 raw[FR];
                float x = 0.f;                    // this lane's share of g . v_i, then the warp's
                if constexpr (LOAD) {
                    if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                    const uint32_t sb = stages_a + (uint32_t)st * pitch;
#pragma unroll
                    for (int k = 0; k < FR; ++k) raw[k] = valid[k] ? lds_v4(sb + foff[k]) : zero4;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_a + 8u * st);
                    if (++st == NS) { st = 0; ph ^= 1u; }
                } else {
#pragma unroll
                    for (int k = 0; k < FR; ++k) raw[k] = zero4;
                }
                float2 a2 = make_float2(0.f, 0.f), b2 = a2;
                if constexpr (ACC) {
                    const uint32_t j4 = (uint32_t)(i - DEPTH) * BT4;
                    float gd = SOLO ? d1 : d2;
                    if (WPT > 1) {
                        gd = 0.f;
                        const uint32_t xa = xch_a + 16u * (((i - 2) & 1) * kBwdMaxNcw + t * WPT);
                        for (int w2 = 0; w2 < WPT; ++w2) gd += lds_f32(xa + 16u * w2);
                    }
                    if (part == 0 && lane == 0) sts_f32(gk + j4, gd);
                    const float pj = lds_f32(tb + j4), rj = lds_f32(tb + tfl4 + j4);
                    const float gp = mass * (gd + lds_f32(tb + 2u * tfl4 + j4));
                    sacc = fmaf(pj, gp, sacc);
                    const float b = pj * rj, a = b * gp;
                    a2 = make_float2(a, a); b2 = make_float2(b, b);
                }
                if constexpr (LOAD) {
                    float2 d2a = make_float2(0.f, 0.f), d2b = make_float2(0.f, 0.f);
                    if constexpr (PACKG && S::kBytes == 2) {
                        // both operands are packed bf16: the dot product straight from the packed registers (the same
                        // four partial sums, in the same order, as the unpacked route below)
#pragma unroll
                        for (int k = 0; k < FR; ++k) {
                            fma_bf16x2(gpk[k].x, raw[k].x, d2a.x, d2a.y);
                            fma_bf16x2(gpk[k].y, raw[k].y, d2b.x, d2b.y);
                            fma_bf16x2(gpk[k].z, raw[k].z, d2a.x, d2a.y);
                            fma_bf16x2(gpk[k].w, raw[k].w, d2b.x, d2b.y);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < FR; ++k) {
                            float2 vf[P], gf[P];
                            S::unpack2(raw[k], vf);
                            load_g(k, gf);
#pragma unroll
                            for (int e = 0; e < P; e += 2) {
                                d2a = __ffma2_rn(gf[e], vf[e], d2a);
                                d2b = __ffma2_rn(gf[e + 1], vf[e + 1], d2b);
                            }
                        }
                    }
                    x = (d2a.x + d2b.x) + (d2a.y + d2b.y);
                }
                // the warp reduction (offsets 16, 8, 4, 2, 1: warp_sum's order) with the accumulation spread between its steps
                constexpr int kShuffles = 5;
#pragma unroll
                for (int k = 0; k < (FR > kShuffles ? FR : kShuffles); ++k) {
                    if constexpr (LOAD) {
                        if (k < kShuffles) x += __shfl_xor_sync(0xffffffffu, x, 16 >> k);
                    }
                    if constexpr (ACC) {
                        if (k < FR) {
                            float2 vf[P];
                            S::unpack2(SOLO ? v1[k] : v2[k], vf);
#pragma unroll
                            for (int e = 0; e < P; ++e) {
                                A[k][e] = __ffma2_rn(a2, vf[e], A[k][e]);
                                B[k][e] = __ffma2_rn(b2, vf[e], B[k][e]);
                            }
                        }
                    }
                }
                if (WPT > 1) named_bar_sync(bar_id, bar_threads);
                if (i < n + DEPTH - 1) {          // after the loop v2 (SOLO: v1) still holds source n - 1 (used by phase 2)
                    d2 = d1; d1 = x;
#pragma unroll
                    for (int k = 0; k < FR; ++k) { if constexpr (!SOLO) v2[k] = v1[k]; v1[k] = raw[k]; }
                }
            };
            if constexpr (!SOLO) {
                // Several warps per token: the sources are taken up to four at a time, in two sweeps over the same ring
                // stages. Sweep 1 forms this warp's share of the group's dot products; their shuffle reductions run
                // interleaved, and the token's warps exchange all the partial sums through ONE barrier (instead of one
                // barrier and one dependent reduction per source). Sweep 2 reads the tiles again from shared memory,
                // accumulates them and releases the stages. A group is at most half the ring, so that the producer
                // fetches the next group meanwhile. Every sum is formed in the order of the one-warp-per-token loops.
                constexpr int GS = 4;
                const int gs = NS >= 2 * GS ? GS : (NS >= 2 ? NS / 2 : 1);
                // (one group, its size a compile-time constant: straight-line code, as in the loops below)
                auto group = [&](int base, int grp, auto m_tag) {
                    constexpr int m = decltype(m_tag)::value;
                    const uint32_t xb = xch_a + 16u * ((grp & 1) * kBwdMaxNcw);
                    float x[GS];
                    uint32_t sbs[GS];
                    {
                        int stj = st; uint32_t phj = ph;
#pragma unroll
                        for (int j = 0; j < GS; ++j) {
                            x[j] = 0.f; sbs[j] = stages_a;
                            if (j < m) {
                                if (alive && !mbar_wait(full_a + 8u * stj, phj, wc, kDevWaitFull)) alive = false;
                                sbs[j] = stages_a + (uint32_t)stj * pitch;
                                if (++stj == NS) { stj = 0; phj ^= 1u; }
                                float2 d2a = make_float2(0.f, 0.f), d2b = make_float2(0.f, 0.f);
#pragma unroll
                                for (int k = 0; k < FR; ++k) {
                                    const uint4 raw = valid[k] ? lds_v4(sbs[j] + foff[k]) : zero4;
                                    if constexpr (PACKG && S::kBytes == 2) {
                                        // both operands are packed bf16: the dot product straight from the packed registers
                                        fma_bf16x2(gpk[k].x, raw.x, d2a.x, d2a.y);
                                        fma_bf16x2(gpk[k].y, raw.y, d2b.x, d2b.y);
                                        fma_bf16x2(gpk[k].z, raw.z, d2a.x, d2a.y);
                                        fma_bf16x2(gpk[k].w, raw.w, d2b.x, d2b.y);
                                    } else {
                                        float2 vf[P], gf[P];
                                        S::unpack2(raw, vf);
                                        load_g(k, gf);
#pragma unroll
                                        for (int e = 0; e < P; e += 2) {
                                            d2a = __ffma2_rn(gf[e], vf[e], d2a);
                                            d2b = __ffma2_rn(gf[e + 1], vf[e + 1], d2b);
                                        }
                                    }
                                }
                                x[j] = (d2a.x + d2b.x) + (d2a.y + d2b.y);
                            }
                        }
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                        for (int j = 0; j < GS; ++j) x[j] += __shfl_xor_sync(0xffffffffu, x[j], o);
                    if (lane == 0) sts_f4(xb + 16u * warp, make_float4(x[0], x[1], x[2], x[3]));
                    named_bar_sync(bar_id, bar_threads);
                    float gd[GS] = {0.f, 0.f, 0.f, 0.f};
                    for (int w2 = 0; w2 < WPT; ++w2) {
                        const float4 q = lds_f4(xb + 16u * (t * WPT + w2));
                        gd[0] += q.x; gd[1] += q.y; gd[2] += q.z; gd[3] += q.w;
                    }
#pragma unroll
                    for (int j = 0; j < GS; ++j) {
                        if (j < m) {
                            const uint32_t j4 = (uint32_t)(base + j) * BT4;
                            if (part == 0 && lane == 0) sts_f32(gk + j4, gd[j]);
                            const float pj = lds_f32(tb + j4), rj = lds_f32(tb + tfl4 + j4);
                            const float gp = mass * (gd[j] + lds_f32(tb + 2u * tfl4 + j4));
                            sacc = fmaf(pj, gp, sacc);
                            const float b = pj * rj, a = b * gp;
                            const float2 a2 = make_float2(a, a), b2 = make_float2(b, b);
#pragma unroll
                            for (int k = 0; k < FR; ++k) {
                                const uint4 raw = valid[k] ? lds_v4(sbs[j] + foff[k]) : zero4;
                                v2[k] = raw;              // after the last group: source n - 1 (used by phase 2)
                                float2 vf[P];
                                S::unpack2(raw, vf);
#pragma unroll
                                for (int e = 0; e < P; ++e) {
                                    A[k][e] = __ffma2_rn(a2, vf[e], A[k][e]);
                                    B[k][e] = __ffma2_rn(b2, vf[e], B[k][e]);
                                }
                            }
                            __syncwarp();
                            if (lane == 0) mbar_arrive(empty_a + 8u * st);
                            if (++st == NS) { st = 0; ph ^= 1u; }
                        }
                    }
                };
                int grp = 0;
                for (int base = 0; base < n; base += gs, ++grp) {
                    switch (min(gs, n - base)) {
                        case 4: group(base, grp, std::integral_constant<int, 4>{}); break;
                        case 3: group(base, grp, std::integral_constant<int, 3>{}); break;
                        case 2: group(base, grp, std::integral_constant<int, 2>{}); break;
                        default: group(base, grp, std::integral_constant<int, 1>{}); break;
                    }
                }
            } else {
                int i = 0;
                for (; i < DEPTH; ++i) {                                   // fill: nothing to accumulate yet
                    if (i < n) iter(i, std::true_type{}, std::false_type{});
                    else iter(i, std::false_type{}, std::false_type{});
                }
                // (unrolled in the deferred form: the register rotation at the end of an iteration disappears into the
                // renaming between the copies; the other forms have no registers to spare for it)
                constexpr int kUnroll = DEFER ? LB_BWD_UNROLL : 1;
#pragma unroll kUnroll
                for (; i < n; ++i) iter(i, std::true_type{}, std::true_type{});      // steady state
                for (; i < n + DEPTH; ++i) iter(i, std::false_type{}, std::true_type{});   // drain
            }
            // ---- query-gradient partial of this thread's columns: private shared-memory slots
            if (alive && tok_in) {
                const float2 ms2 = make_float2(-sacc, -sacc);
#pragma unroll
                for (int k = 0; k < FR; ++k)
#pragma unroll
                    for (int e4 = 0; e4 < V4; ++e4) {
                        const uint32_t sa = slots_a + (uint32_t)((k * V4 + e4) * kConsumerThreads + threadIdx.x) * 16u;
                        float4 s4 = lds_f4(sa);
                        const float2 lo = __ffma2_rn(ms2, B[k][2 * e4], A[k][2 * e4]);
                        const float2 hi = __ffma2_rn(ms2, B[k][2 * e4 + 1], A[k][2 * e4 + 1]);
                        s4.x += lo.x; s4.y += lo.y; s4.z += hi.x; s4.w += hi.y;
                        sts_f4(sa, s4);
                    }
            }
            // ---- per-source scalars of this token: lanes over sources, by the token's first warp
            __syncwarp();
            if (part == 0) {
                for (int i = lane; i < n; i += 32) {
                    const uint32_t i4 = (uint32_t)i * BT4;
                    const float gd = lds_f32(gk + i4);
                    const float pi = lds_f32(tb + i4), ri = lds_f32(tb + tfl4 + i4);
                    const float gp = mass * (gd + lds_f32(tb + 2u * tfl4 + i4));
                    const float dz = pi * (gp - sacc);
                    sts_f32(gk + i4, dz * ri * inv);
                    const float drtot = lds_f32(tb + 5u * tfl4 + i4) + dz * lds_f32(tb + 4u * tfl4 + i4);
                    if (p.finalize && i == n - 1) sts_f32(fin_a + t4, drtot * (-(ri * ri * ri)) / (float)p.d);
                    if constexpr (DEFER) {
                        if (fin2 && i == 0) sts_f32(fin0_a + t4, drtot * (-(ri * ri * ri)) / (float)p.d);
                        if (alive && tok_in && i < n - 1) {
                            // what the later finishing of update i needs of this step: its coefficient of g and of q
                            const long long e = ((long long)(n - 1) * p.n_total + i) * p.n_tok + tok;
                            p.Wt[e] = lds_f32(tb + 3u * tfl4 + i4);
                            p.KQt[e] = dz * ri * inv;
                        }
                    }
                    if (alive && tok_in) {
                        p.dR[(long long)i * p.n_tok + tok] = drtot;
                        if (p.tc_prev == nullptr) p.dcbar[tok * n + i] = -gd;
                        else if (i < n - 1) p.dcbar[tok * (n - 1) + i] = -(p.lam * gd);      // d/d tc_prev
                    }
                }
            }
            if (WPT > 1) named_bar_sync(bar_id, bar_threads); else __syncwarp();

            // ---- phase 2: the gradient of every source
            // (the step's own query row: held in registers where every source's update uses it; the deferred form uses it
            // once per finished update and reads it where it is used)
            auto load_q = [&](int k, float2 (&qf)[P]) {
                const int col = (chunk0 + k) * BW + lane * VEC;
#pragma unroll
                for (int e4 = 0; e4 < V4; ++e4) {
                    const float4 q4 = lds_f4(qsm_a + 16u * (col / 4 + e4));
                    qf[2 * e4] = make_float2(q4.x, q4.y);
                    qf[2 * e4 + 1] = make_float2(q4.z, q4.w);
                }
            };
            float2 q2[DEFER ? 1 : FR][P];
            if constexpr (!DEFER) {
#pragma unroll
                for (int k = 0; k < FR; ++k) load_q(k, q2[k]);
            }
            if constexpr (DEFER) {
                // The finished gradient of an update, formed in one go:
                //   dV = sum over the steps s' that read it (this one, then the J that ran their backward before it) of
                //        w_{s'} g_{s'} + kq_{s'} q_{s'},   plus its key-scale term,
                // accumulated in fp32 and rounded once. g_{s'} comes from the g stack through the ring, the two scalars
                // from the tables the scalar warps prepared, the query row from global memory (one tile ahead).
                const uint32_t ftb = ft_a + buf * 4u * ftl4 + t4;
                auto finish = [&](auto main_tag, int src, uint32_t ftab, const uint4 (&vfr)[FR], float kf) {
                    constexpr bool MAIN = decltype(main_tag)::value;
                    const uint32_t s4 = (uint32_t)src * BT4;
                    const float w_own = lds_f32(tb + 3u * tfl4 + s4), kq_own = lds_f32(gk + s4);
                    const float2 w2 = make_float2(w_own, w_own), kq2 = make_float2(kq_own, kq_own), kf2 = make_float2(kf, kf);
                    float2 acc[FR][P];
#pragma unroll
                    for (int k = 0; k < FR; ++k) {
                        float2 gf[P], vf[P], qf[P];
                        load_g(k, gf);
                        load_q(k, qf);
                        S::unpack2(vfr[k], vf);
#pragma unroll
                        for (int e = 0; e < P; ++e)
                            acc[k][e] = __ffma2_rn(kf2, vf[e], __ffma2_rn(w2, gf[e], __fmul2_rn(kq2, qf[e])));
                    }
                    for (int j = 0; j < J; ++j) {
                        if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                        const uint32_t sb = stages_a + (uint32_t)st * pitch;
                        const float fw = lds_f32(ftab + (uint32_t)j * BT4), fkq = lds_f32(ftab + ftl4 + (uint32_t)j * BT4);
                        const float2 fw2 = make_float2(fw, fw), fkq2 = make_float2(fkq, fkq);
#pragma unroll
                        for (int k = 0; k < FR; ++k) {
                            float2 gf[P];
                            S::unpack2(valid[k] ? lds_v4(sb + foff[k]) : zero4, gf);
                            // the query row arrives permuted (lb_permute_queries): per chunk, quarter e4 of every lane's
                            // columns is contiguous over the lanes, so these 128-bit reads are conflict-free
                            const uint32_t qa = sb + kStageBytes + (uint32_t)(chunk0 + k) * (uint32_t)(BW * 4) + 16u * lane;
#pragma unroll
                            for (int e4 = 0; e4 < V4; ++e4) {
                                const float4 q4 = valid[k] ? lds_f4(qa + 512u * e4) : make_float4(0.f, 0.f, 0.f, 0.f);
                                acc[k][2 * e4] = __ffma2_rn(fkq2, make_float2(q4.x, q4.y), acc[k][2 * e4]);
                                acc[k][2 * e4 + 1] = __ffma2_rn(fkq2, make_float2(q4.z, q4.w), acc[k][2 * e4 + 1]);
                            }
#pragma unroll
                            for (int e = 0; e < P; ++e) acc[k][e] = __ffma2_rn(fw2, gf[e], acc[k][e]);
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty_a + 8u * st);
                        if (++st == NS) { st = 0; ph ^= 1u; }
                    }
#pragma unroll
                    for (int k = 0; k < FR; ++k) {
                        const uint4 res = S::pack2v(acc[k]);
                        const int col = (chunk0 + k) * BW + lane * VEC;
                        const bool live = alive && tok_in && col < p.d;
                        const long long off = tok * (long long)p.d + col;
                        if constexpr (MAIN) {
                            if (live) st_global_v4(reinterpret_cast<T *>(p.neg_out) + off, S::negate(res));
                            float2 gf[P];
                            load_g(k, gf);
                            if (p.blend) {
                                const float2 b2 = make_float2(p.beta, p.beta);
                                float2 bg[P];
#pragma unroll
                                for (int e = 0; e < P; ++e) bg[e] = __fmul2_rn(b2, gf[e]);
                                S::unpack2(S::pack2v(bg), bg);                  // rounded to the storage type
#pragma unroll
                                for (int e = 0; e < P; ++e) gf[e] = __fadd2_rn(gf[e], make_float2(-bg[e].x, -bg[e].y));
                            }
                            if (live) st_global_v4(reinterpret_cast<T *>(p.dh_out) + off, S::accum(res, gf));
                        } else {
                            if (live) {
                                st_global_v4(reinterpret_cast<T *>(p.dv0_out) + off, res);
                                st_global_v4(reinterpret_cast<T *>(p.neg0_out) + off, S::negate(res));
                            }
                        }
                    }
                };
                finish(std::true_type{}, n - 1, ftb, SOLO ? v1 : v2, lds_f32(fin_a + t4));
                if (fin2) {
                    // update 0 has no step of its own: its fragments come back through the ring, then the same rows of g again
                    if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                    const uint32_t sb = stages_a + (uint32_t)st * pitch;
                    uint4 v0f[FR];
#pragma unroll
                    for (int k = 0; k < FR; ++k) v0f[k] = valid[k] ? lds_v4(sb + foff[k]) : zero4;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_a + 8u * st);
                    if (++st == NS) { st = 0; ph ^= 1u; }
                    finish(std::false_type{}, 0, ftb + 2u * ftl4, v0f, lds_f32(fin0_a + t4));
                }
            } else if constexpr (STEP) {
                T *dvrow = reinterpret_cast<T *>(p.dV) + tok * (long long)p.d + chunk0 * BW + lane * VEC;
                const long long src_stride = p.n_tok * (long long)p.d;
                // One source of phase 2. FINAL (compile time) is the newest source of a finalising read, peeled out of the
                // loop over the older sources so that the loop body carries none of its extra outputs.
                auto phase2_source = [&](int i, auto final_tag) {
                    constexpr bool FINAL = decltype(final_tag)::value;
                    const uint32_t i4 = (uint32_t)i * BT4;
                    const float wi = lds_f32(tb + 3u * tfl4 + i4), kq = lds_f32(gk + i4);
                    const float2 w2 = make_float2(wi, wi), kq2 = make_float2(kq, kq);
                    uint4 prev[FR];
                    if (p.accum) {
                        if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                        const uint32_t sb = stages_a + (uint32_t)st * pitch;
#pragma unroll
                        for (int k = 0; k < FR; ++k) prev[k] = valid[k] ? lds_v4(sb + foff[k]) : zero4;
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty_a + 8u * st);
                        if (++st == NS) { st = 0; ph ^= 1u; }
                    }
#pragma unroll
                    for (int k = 0; k < FR; ++k) {
                        float2 o[P], gf[P];
                        load_g(k, gf);
#pragma unroll
                        for (int e = 0; e < P; ++e) o[e] = __ffma2_rn(w2, gf[e], __fmul2_rn(kq2, q2[k][e]));
                        uint4 res = p.accum ? S::accum(prev[k], o) : S::pack2v(o);
                        const int col = (chunk0 + k) * BW + lane * VEC;
                        const bool live = alive && tok_in && col < p.d;
                        if constexpr (FINAL) {
                            // this read is the last to touch source n-1: add the gradient that reaches the update through
                            // its key scale, dR (-r^3/d) v, rounded like the separate accumulation kernel would, and hand
                            // out the negated total (the gradient of the block input)
                            const float kf = lds_f32(fin_a + t4);
                            const float2 kf2 = make_float2(kf, kf);
                            {
                                float2 kv[P];
                                S::unpack2(SOLO ? v1[k] : v2[k], kv);
#pragma unroll
                                for (int e = 0; e < P; ++e) kv[e] = __fmul2_rn(kf2, kv[e]);
                                res = S::accum(res, kv);
                            }
                            const long long off = tok * (long long)p.d + col;
                            if (live) st_global_v4(reinterpret_cast<T *>(p.neg_out) + off, S::negate(res));
                            {
                                // the gradient of the block output: the update's finished gradient plus what reaches it as
                                // the read's base -- g itself inside an iteration; at an iteration's end, where
                                // base = h + beta (h0 - h), autograd's round(g - round(beta g))
                                if (p.blend) {
                                    const float2 b2 = make_float2(p.beta, p.beta);
                                    float2 bg[P];
#pragma unroll
                                    for (int e = 0; e < P; ++e) bg[e] = __fmul2_rn(b2, gf[e]);
                                    S::unpack2(S::pack2v(bg), bg);                  // rounded to the storage type
#pragma unroll
                                    for (int e = 0; e < P; ++e) gf[e] = __fadd2_rn(gf[e], make_float2(-bg[e].x, -bg[e].y));
                                }
                                if (live) st_global_v4(reinterpret_cast<T *>(p.dh_out) + off, S::accum(res, gf));
                            }
                            // (the finished gradient itself is not stored: no later backward reads it)
                        } else {
                            if (live) st_global_v4(dvrow + k * BW, res);
                        }
                    }
                    if constexpr (!FINAL) dvrow += src_stride;
                };
                // One warp per token: the finished source first, which frees the registers that hold its fragments for
                // the loop over the older ones. Several warps per token: last, as in the plain kernel (measured: the
                // other order costs those shapes 3 %, and this one costs the one-warp shape 6 %).
                if constexpr (SOLO) phase2_source(n - 1, std::true_type{});
                for (int i = 0; i < n - 1; ++i) phase2_source(i, std::false_type{});
                if constexpr (!SOLO) phase2_source(n - 1, std::true_type{});
            } else {
                T *dvrow = reinterpret_cast<T *>(p.dV) + tok * (long long)p.d + chunk0 * BW + lane * VEC;
                const long long src_stride = p.n_tok * (long long)p.d;
                for (int i = 0; i < n; ++i) {
                    const uint32_t i4 = (uint32_t)i * BT4;
                    const float wi = lds_f32(tb + 3u * tfl4 + i4), kq = lds_f32(gk + i4);
                    const float2 w2 = make_float2(wi, wi), kq2 = make_float2(kq, kq);
                    uint4 prev[FR];
                    if (p.accum) {
                        if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                        const uint32_t sb = stages_a + (uint32_t)st * pitch;
#pragma unroll
                        for (int k = 0; k < FR; ++k) prev[k] = valid[k] ? lds_v4(sb + foff[k]) : zero4;
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty_a + 8u * st);
                        if (++st == NS) { st = 0; ph ^= 1u; }
                    }
#pragma unroll
                    for (int k = 0; k < FR; ++k) {
                        float2 o[P], gf[P];
                        load_g(k, gf);
#pragma unroll
                        for (int e = 0; e < P; ++e) o[e] = __ffma2_rn(w2, gf[e], __fmul2_rn(kq2, q2[k][e]));
                        uint4 res = p.accum ? S::accum(prev[k], o) : S::pack2v(o);
                        const int col = (chunk0 + k) * BW + lane * VEC;
                        if (p.finalize && i == n - 1) {
                            // this read is the last to touch source n-1: add the gradient that reaches the update through
                            // its key scale, dR (-r^3/d) v, rounded like the separate accumulation kernel would, and hand
                            // out the negated total (the gradient of the block input)
                            const float kf = lds_f32(fin_a + t4);
                            const float2 kf2 = make_float2(kf, kf);
                            float2 vf[P], kv[P];
                            S::unpack2(SOLO ? v1[k] : v2[k], vf);
#pragma unroll
                            for (int e = 0; e < P; ++e) kv[e] = __fmul2_rn(kf2, vf[e]);
                            res = S::accum(res, kv);
                            if (p.neg_out != nullptr && alive && tok_in && col < p.d)
                                st_global_v4(reinterpret_cast<T *>(p.neg_out) + tok * (long long)p.d + col, S::negate(res));
                        }
                        if (alive && tok_in && col < p.d) st_global_v4(dvrow + k * BW, res);
                    }
                    dvrow += src_stride;
                }
            }
            // the token's warps leave the tile together: gdkq and xch are reused by the next tile
            if (WPT > 1) named_bar_sync(bar_id, bar_threads); else __syncwarp();
            if (lane == 0) mbar_arrive(sempty_a + 8u * buf);
        }
        // ---- the CTA's query-gradient row: sum the private slots over the tile's tokens
        named_bar_sync(15, kConsumerThreads);
        if (t == 0) {
#pragma unroll
            for (int k = 0; k < FR; ++k) {
                const int col = (chunk0 + k) * BW + lane * VEC;
#pragma unroll
                for (int e4 = 0; e4 < V4; ++e4) {
                    float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int t2 = 0; t2 < BT; ++t2) {
                        const float4 v4 = lds_f4(slots_a + (uint32_t)((k * V4 + e4) * kConsumerThreads +
                                                                      (t2 * WPT + part) * 32 + lane) * 16u);
                        s4.x += v4.x; s4.y += v4.y; s4.z += v4.z; s4.w += v4.w;
                    }
                    if (col < p.d)
                        *reinterpret_cast<float4 *>(p.dq_part + (long long)blockIdx.x * p.d + col + 4 * e4) = s4;
                }
            }
        }
    } else if (warp == NCW) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            tma_prefetch_desc(&tmV);
            tma_prefetch_desc(&tmG);
            if (p.accum || DEFER) tma_prefetch_desc(&tmDV);
            if (dh0_rmw) tma_prefetch_desc(&tmH0);
            const int v0 = dh0_rmw ? 2 : 1;                      // first V item; item 1 is the h0-gradient tile if any
            // the order in which phase 2 wants the old gradients: a finalising read takes the newest source first
            // which slice of the second stack an item past the sources asks for. Plain / step: the old gradient of source
            // j, a one-warp-per-token step taking the newest first. Deferred: the g row of the j-th earlier backward step
            // (slice n + j), and after update 0's fragments (item J) the same rows once more.
            auto dv_source = [&](int j) {
                if (DEFER) return n + (j > J ? j - J - 1 : j);
                return MODE == 1 && SOLO ? (j == 0 ? n - 1 : j - 1) : j;
            };
            int st = 0; uint32_t ph = 0;
            int issued = 0;
            bool ok = true;
            const int nch = p.chunks;                       // the full row
            for (long long tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const int tok0 = (int)(tile * BT);
                for (int item = 0; item < items_per_tile; ++item) {
                    if (!mbar_wait(empty_a + 8u * st, ph ^ 1u, wc, kDevWaitEmpty)) {
                        ok = false;
                        break;
                    }
                    const uint32_t sb = stages_a + (uint32_t)st * pitch, fb = full_a + 8u * st;
                    // deferred form: which earlier backward step a g item belongs to (-1: not a g item)
                    int gj = -1;
                    if (DEFER && item >= v0 + n && item != v0 + n + J) gj = item - v0 - n - (item > v0 + n + J ? J + 1 : 0);
                    mbar_arrive_expect_tx(fb, (uint32_t)(nch * BT * kChunkBytes) + (gj >= 0 ? (uint32_t)p.qrow_bytes : 0u));
                    if (gj >= 0)        // the query of step n + gj (row n - 1 + gj) rides behind the tile
                        bulk_load(sb + kStageBytes, p.Qall + (long long)(n - 1 + gj) * (p.qrow_bytes / 4), (uint32_t)p.qrow_bytes, fb);
                    if (p.rank4) {
                        if (item == 0) tma_load_3d(sb, &tmG, fb, 0, 0, tok0);
                        else if (item < v0) tma_load_3d(sb, &tmH0, fb, 0, 0, tok0);
                        else if (item < v0 + n) tma_load_4d(sb, &tmV, fb, 0, 0, tok0, item - v0);
                        else if (DEFER && item == v0 + n + J) tma_load_4d(sb, &tmV, fb, 0, 0, tok0, 0);
                        else tma_load_4d(sb, &tmDV, fb, 0, 0, tok0, dv_source(item - v0 - n));
                    } else {
                        for (int c = 0; c < nch; ++c) {
                            const uint32_t dst = sb + (uint32_t)(c * BT * kChunkBytes);
                            if (item == 0) tma_load_2d(dst, &tmG, fb, c * BW, tok0);
                            else if (item < v0) tma_load_2d(dst, &tmH0, fb, c * BW, tok0);
                            else if (item < v0 + n) tma_load_3d(dst, &tmV, fb, c * BW, tok0, item - v0);
                            else if (DEFER && item == v0 + n + J) tma_load_3d(dst, &tmV, fb, c * BW, tok0, 0);
                            else tma_load_3d(dst, &tmDV, fb, c * BW, tok0, dv_source(item - v0 - n));
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
        // ------------------------------------------------------------------ scalar warps: tables of the next tile
        const int sw = warp - NCW - 1;
        const float mass = lds_f32(mass_a);
        int tcount = 0;
        for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tcount) {
            const uint32_t buf = tcount & 1;
            if (!mbar_wait<true>(sempty_a + 8u * buf, (uint32_t)(((tcount >> 1) & 1) ^ 1), wc, kDevWaitScalarSlot))
                return;
            const uint32_t tb = tables_a + buf * kBwdTables * tfl4;
            // (the loads of up to four passes over the tile's (token, source) pairs are all requested before the first
            // is used: one memory round trip per tile instead of one per pass -- this is what a launch's first tile waits for)
            constexpr int SU = 4;
            constexpr int kStride = kBwdScalarWarps * 32;
            for (int idx0 = sw * 32 + lane; idx0 < BT * n; idx0 += SU * kStride) {
                float lgv[SU], lsev[SU], lse0v[SU], cbv[SU], gtvv[SU], rv[SU], drpv[SU];
#pragma unroll
                for (int u = 0; u < SU; ++u) {
                    const int idx = idx0 + u * kStride;
                    lgv[u] = 0.f; lsev[u] = 0.f; lse0v[u] = 0.f; cbv[u] = 0.f; gtvv[u] = 0.f; rv[u] = 1.f; drpv[u] = 0.f;
                    if (idx < BT * n) {
                        const int t = idx / n, i = idx - t * n;
                        long long tok = tile * BT + t;
                        if (tok >= p.n_tok) tok = p.n_tok - 1;
                        lgv[u] = __ldg(p.LG + tok * n + i);
                        lsev[u] = __ldg(p.LSE + tok); lse0v[u] = __ldg(p.LSE0 + tok);
                        cbv[u] = p.tc_prev == nullptr ? __ldg(p.cbar + tok * n + i)
                                                      : (i < n - 1 ? p.lam * __ldg(p.tc_prev + tok * (n - 1) + i) : p.lam);
                        gtvv[u] = p.gt ? __ldg(p.gt + tok * n + i) : 0.f;
                        rv[u] = __ldg(p.R + (long long)i * p.n_tok + tok);
                        drpv[u] = p.accum ? p.dR[(long long)i * p.n_tok + tok] : 0.f;
                    }
                }
#pragma unroll
                for (int u = 0; u < SU; ++u) {
                    const int idx = idx0 + u * kStride;
                    if (idx < BT * n) {
                        const int t = idx / n, i = idx - t * n;
                        const float lg = lgv[u], r = rv[u];
                        const float lci = lds_f32(lc_a + 4u * i);
                        const float pi = expf(lg - lsev[u]), p0 = expf(lci - lse0v[u]);
                        const uint32_t o = tb + 4u * (uint32_t)(i * BT + t);
                        sts_f32(o, pi);
                        sts_f32(o + tfl4, r);
                        sts_f32(o + 2u * tfl4, gtvv[u]);
                        sts_f32(o + 3u * tfl4, lds_f32(c0_a + 4u * i) - cbv[u] + mass * (pi - p0));
                        sts_f32(o + 4u * tfl4, (lg - lci) / r);
                        sts_f32(o + 5u * tfl4, drpv[u]);
                    }
                }
            }
            if constexpr (DEFER) {
                // the scalars the earlier backward steps left for the update(s) this step finishes: lanes over tokens
                const uint32_t ft = ft_a + buf * 4u * ftl4;
                for (int idx0 = sw * 32 + lane; idx0 < BT * J; idx0 += SU * kStride) {
                    float wv[SU], kv[SU], w0v[SU], k0v[SU];
#pragma unroll
                    for (int u = 0; u < SU; ++u) {
                        const int idx = idx0 + u * kStride;
                        wv[u] = 0.f; kv[u] = 0.f; w0v[u] = 0.f; k0v[u] = 0.f;
                        if (idx < BT * J) {
                            const int j = idx / BT, t = idx - j * BT;
                            long long tok = tile * BT + t;
                            if (tok >= p.n_tok) tok = p.n_tok - 1;
                            const long long e = ((long long)(n + j) * p.n_total + (n - 1)) * p.n_tok + tok;
                            wv[u] = __ldg(p.Wt + e); kv[u] = __ldg(p.KQt + e);
                            if (fin2) {
                                const long long e0 = (long long)(n + j) * p.n_total * p.n_tok + tok;
                                w0v[u] = __ldg(p.Wt + e0); k0v[u] = __ldg(p.KQt + e0);
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < SU; ++u) {
                        const int idx = idx0 + u * kStride;
                        if (idx < BT * J) {
                            sts_f32(ft + 4u * (uint32_t)idx, wv[u]);
                            sts_f32(ft + ftl4 + 4u * (uint32_t)idx, kv[u]);
                            if (fin2) {
                                sts_f32(ft + 2u * ftl4 + 4u * (uint32_t)idx, w0v[u]);
                                sts_f32(ft + 3u * ftl4 + 4u * (uint32_t)idx, k0v[u]);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(sfull_a + 8u * buf);
        }
    }
}

template <typename T, int FR, int NCW, bool SOLO, int MODE>
static cudaError_t launch_bwd(const CUtensorMap &tmV, const CUtensorMap &tmG, const CUtensorMap &tmDV,
                              const CUtensorMap &tmH0, const ReadBwdParams &p, int grid, cudaStream_t stream) {
    size_t smem = read_bwd_smem_bytes(FR, NCW, p.wpt, p.stages, p.n, Store<T>::kVec, MODE == 2 ? p.n_total - p.n : 0,
                                      MODE == 2 ? p.qrow_bytes : 0);
    cudaError_t e = cudaFuncSetAttribute(read_bwd_kernel<T, FR, NCW, SOLO, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    read_bwd_kernel<T, FR, NCW, SOLO, MODE><<<grid, (NCW + 1 + bwd_scalar_warps(NCW)) * 32, smem, stream>>>(tmV, tmG, tmDV, tmH0, p);
    return cudaGetLastError();
}

// The instantiated shapes of one storage type. Several warps per token: 16 consumer warps x {1,2} fragments, 12 x {1,2},
// 8 x {1,2,3,4}; one warp per token (SOLO): 8 x {1,2,3,4} and the half-size 4 x {1,2,3,4}. Each storage type has a
// translation unit of its own (lb_read_bwd.cu: bf16, lb_read_bwd_f32.cu: fp32), so that they compile side by side.
template <typename TT>
static cudaError_t launch_read_bwd_typed(int fr, int ncw, const CUtensorMap &tmV, const CUtensorMap &tmG,
                                         const CUtensorMap &tmDV, const CUtensorMap &tmH0, const ReadBwdParams &p, int grid,
                                         cudaStream_t stream) {
#define LB_BWD_CASE(F, W, SOLO_) \
    if (fr == F && ncw == W && (p.wpt == 1) == SOLO_)                                                             \
        return p.Gst    ? launch_bwd<TT, F, W, SOLO_, 2>(tmV, tmG, tmDV, tmH0, p, grid, stream)                     \
             : p.dh_out ? launch_bwd<TT, F, W, SOLO_, 1>(tmV, tmG, tmDV, tmH0, p, grid, stream)                     \
                        : launch_bwd<TT, F, W, SOLO_, 0>(tmV, tmG, tmDV, tmH0, p, grid, stream);
    LB_BWD_CASE(1, 16, false) LB_BWD_CASE(2, 16, false) LB_BWD_CASE(1, 12, false)
    LB_BWD_CASE(2, 12, false) LB_BWD_CASE(1, 8, false) LB_BWD_CASE(2, 8, false)
    LB_BWD_CASE(3, 8, false) LB_BWD_CASE(4, 8, false) LB_BWD_CASE(1, 8, true) LB_BWD_CASE(2, 8, true)
    LB_BWD_CASE(3, 8, true) LB_BWD_CASE(4, 8, true)
    LB_BWD_CASE(1, 4, true) LB_BWD_CASE(2, 4, true) LB_BWD_CASE(3, 4, true) LB_BWD_CASE(4, 4, true)
#undef LB_BWD_CASE
    return cudaErrorInvalidValue;
}

cudaError_t launch_read_bwd_f32(int fr, int ncw, const CUtensorMap &tmV, const CUtensorMap &tmG, const CUtensorMap &tmDV,
                                const CUtensorMap &tmH0, const ReadBwdParams &p, int grid, cudaStream_t stream);

}  // namespace lb
