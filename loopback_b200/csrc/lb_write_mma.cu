// Update write for training-sized batches of bf16 rows (sm_100a): persistent, TMA-fed, scores on the tensor cores.
//
// Replaces the reference's _write_stk_kernel (fused_dattn.py:561-585) where the batch is large enough to give every
// SM a tile of its own:  V[s] = round(h - x),  R[s] = rsqrt(mean(V[s]^2) + eps),  DOTS[j][s][t] = q_j . V[s][t]
// for the queries j0 <= j < j0 + nq whose reads will see update s.
//
// The scores are the one contraction on the whole path ([tokens x d] . [d x nq]); on the fp32 pipes they cost more
// issue slots than the row traffic leaves room for. Here they run as bf16 mma with fp32 accumulation, the fp32 query
// split into three bf16 terms (q = hi + mid + lo, 24 mantissa bits in all), so every product is exact and the sums
// are fp32 as in the reference.
//
// One CTA per SM; a CTA owns tiles of up to 256 consecutive tokens and walks each tile's rows in chunks of 64 columns:
//   * one producer lane fills a ring of stages with the tile's h and x chunk (two TMA boxes of tile_tok x 128 bytes,
//     128-byte swizzle so that the 16-byte accesses of 8 rows at one column are conflict-free);
//   * two query warps convert the next chunk of the nq queries into the three bf16 terms (same swizzle), double-buffered;
//   * 8 consumer warps own 32 tokens each (two 16-token mma tiles). Per chunk a lane reads 16-byte fragments of h and x
//     in the mma operand arrangement, subtracts, rounds, stores V, and uses the rounded registers as the A operand as
//     they are (no ldmatrix, nothing written back to shared memory); accumulators stay in registers across the whole
//     row. No CTA-wide barrier.
// Waits are bounded (lb_common.cuh); a CTA that gives up unwinds and reports through the device error word.
#include <type_traits>

#include "lb_common.cuh"
#include "lb_kernels.h"

namespace lb {

constexpr int kWmQueryWarps = 2;
// MT = 16-token mma tiles per consumer warp (1 or 2); 16 / MT consumer warps cover a tile of up to 256 tokens
constexpr int wm_consumers(int mt) { return 16 / mt; }
constexpr int wm_threads(int mt) { return (wm_consumers(mt) + 1 + kWmQueryWarps) * 32; }      // + producer + query warps
constexpr int kWmKC = 64;                                // columns per chunk
constexpr int kWmRow = 128;                              // bytes per token and chunk (one swizzle span)
constexpr int kWmEpPitch = 33;                           // floats per query row of a warp's transposing buffer

__device__ __forceinline__ void sts_v2(uint32_t a, uint32_t x, uint32_t y) {
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// (h - x) for two bf16 pairs: the exact difference rounded once to bf16 (the same value as an fp32 subtraction
// followed by the rounding of a bf16 store)
__device__ __forceinline__ uint32_t bsub2(uint32_t h, uint32_t x) {
    const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&h), *reinterpret_cast<const __nv_bfloat162 *>(&x));
    return *reinterpret_cast<const uint32_t *>(&r);
}

// q = hi + mid + lo with three bf16 terms: each remainder is exact in fp32, the third term carries bits 17..24
__device__ __forceinline__ void split3(float q, uint32_t &hi, uint32_t &mid, uint32_t &lo) {
    const __nv_bfloat16 h = __float2bfloat16_rn(q);
    const float r1 = q - __bfloat162float(h);
    const __nv_bfloat16 m = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(m);
    const __nv_bfloat16 l = __float2bfloat16_rn(r2);
    hi = __bfloat16_as_ushort(h); mid = __bfloat16_as_ushort(m); lo = __bfloat16_as_ushort(l);
}

struct WmBars {
    unsigned long long full[8], empty[8], qfull[2], qempty[2];
    int abort_flag;
    int qlow[2][kWmQueryWarps];      // per query buffer and query warp: does the chunk have a non-zero mid or lo term?
};

// Dynamic shared memory, from a 1024-byte boundary: stages x (h tile | x tile), 2 x 3 query-term blocks of NT x 1024
// bytes, 8 transposing buffers, the barriers.
template <int NT, int MT>
__global__ void __launch_bounds__(wm_threads(MT), 1)
write_mma_kernel(const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmX, WriteMmaParams p) {
    using S = Store<__nv_bfloat16>;
    constexpr int kWmConsumers = wm_consumers(MT);
    constexpr int RW = 16 * MT;                 // rows per consumer warp
    extern __shared__ unsigned char smem_raw[];
    const uint32_t stages_a = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tile_bytes = (uint32_t)p.tile_tok * kWmRow;
    const uint32_t stage_bytes = 2u * tile_bytes;
    constexpr uint32_t kQTerm = (NT > 0 ? NT : 1) * 1024u;          // one bf16 term of one chunk: NT * 8 rows x 128 B
    const uint32_t qs_a = stages_a + (uint32_t)p.stages * stage_bytes;
    const uint32_t ep_a = qs_a + 6u * kQTerm;
    const uint32_t bars_a = ep_a + kWmConsumers * 8u * kWmEpPitch * 4u;
    const uint32_t full_a = bars_a + offsetof(WmBars, full), empty_a = bars_a + offsetof(WmBars, empty);
    const uint32_t qfull_a = bars_a + offsetof(WmBars, qfull), qempty_a = bars_a + offsetof(WmBars, qempty);
    const uint32_t abort_a = bars_a + offsetof(WmBars, abort_flag);
    const uint32_t qlow_a = bars_a + offsetof(WmBars, qlow);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NS = p.stages;
    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full_a + 8u * s, 1); mbar_init(empty_a + 8u * s, kWmConsumers); }
        for (int b = 0; b < 2; ++b) { mbar_init(qfull_a + 8u * b, 32 * kWmQueryWarps); mbar_init(qempty_a + 8u * b, kWmConsumers); }
        sts_s32(abort_a, 0);
        fence_mbar_init();
    }
    __syncthreads();
    const WaitCtx wc{abort_a, p.err_word, p.wait_cycles};
    const int chunks = p.chunks;
    const int nq = NT > 0 ? p.nq : 0;

    if (warp < kWmConsumers) {
        // ------------------------------------------------------------------ consumers
        const int row0 = warp * RW;
        const bool active = row0 < p.tile_tok;           // tiles are whole multiples of 32 tokens
        const uint32_t my_ep = ep_a + (uint32_t)warp * 8u * kWmEpPitch * 4u;
        const int g = lane >> 2, t4 = lane & 3;
        int st = 0; uint32_t ph = 0;
        int qb = 0; uint32_t qph = 0;
        bool alive = true;
        for (long long tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x) {
            const long long tok0 = tile * p.tile_tok;
            float acc[MT][NT > 0 ? NT : 1][4];
            // sums of squares of the rounded update, per 16-token tile: [0..1] rows g (the two diagonal candidates of the
            // rows 0-7 block), [2..3] rows g + 8; only the lane that holds a row's diagonal element uses its value
            float ss[MT][4];
#pragma unroll
            for (int mi = 0; mi < MT; ++mi) {
#pragma unroll
                for (int e = 0; e < 4; ++e) ss[mi][e] = 0.f;
#pragma unroll
                for (int nt = 0; nt < (NT > 0 ? NT : 1); ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[mi][nt][e] = 0.f;
            }
            for (int c = 0; c < chunks; ++c) {
                if (alive && !mbar_wait(full_a + 8u * st, ph, wc, kDevWaitFull)) alive = false;
                if (NT > 0 && alive && !mbar_wait(qfull_a + 8u * qb, qph, wc, kDevWaitScalars)) alive = false;
                const uint32_t sh = stages_a + (uint32_t)st * stage_bytes, sx = sh + tile_bytes;
                // The chunk's work, specialised at compile time on the number of query terms (a chunk whose queries are
                // exact in bf16, e.g. a bf16 parameter, has zero mid and lo terms), so that its loads, subtractions,
                // stores and mma steps are one straight-line block the scheduler can interleave freely.
                auto chunk_body = [&](auto terms_tag) {
                    constexpr int terms = decltype(terms_tag)::value;
                    // Both mma operands come straight from 16-byte shared-memory reads: lane (g, t4) owns fragment
                    // t4 of a 32-column group for rows g and g + 8 of each 16-token tile. Its 8 columns feed two mma
                    // steps (columns 0-3, then 4-7, as the k pairs {2 t4, 2 t4 + 1} and {2 t4 + 8, 2 t4 + 9}); the
                    // query terms are read with the same pattern, so the two operands agree on which column is which k.
                    // The update is formed in bf16 pairs (one exact subtraction, one rounding: what the fp32 route
                    // gives) and goes to HBM and into the mma as it is. Its squares are summed on the tensor cores as
                    // well: with B = the A registers of rows 0-7 (8-15) the product's diagonal is sum_k v[r][k]^2.
                    float part[MT][NT > 0 ? NT : 1][4], sl[MT][4], shh[MT][4];
#pragma unroll
                    for (int mi = 0; mi < MT; ++mi) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) { sl[mi][e] = 0.f; shh[mi][e] = 0.f; }
#pragma unroll
                        for (int nt = 0; nt < (NT > 0 ? NT : 1); ++nt)
#pragma unroll
                            for (int e = 0; e < 4; ++e) part[mi][nt][e] = 0.f;
                    }
                    const uint32_t qbase = qs_a + (uint32_t)qb * 3u * kQTerm;
#pragma unroll
                    for (int grp = 0; grp < kWmKC / 32; ++grp) {
                        const uint32_t unit = (uint32_t)(((4 * grp + t4) ^ g) << 4);      // swizzled; row & 7 == g
                        const int col = c * kWmKC + grp * 32 + t4 * 8;
                        uint32_t afr[2][MT][4];
#pragma unroll
                        for (int mi = 0; mi < MT; ++mi) {
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh) {
                                const int r = row0 + 16 * mi + 8 * hh + g;
                                const uint32_t a = (uint32_t)r * kWmRow + unit;
                                const uint4 hv = lds_v4(sh + a), xv = lds_v4(sx + a);
                                const uint4 packed = make_uint4(bsub2(hv.x, xv.x), bsub2(hv.y, xv.y), bsub2(hv.z, xv.z),
                                                                bsub2(hv.w, xv.w));
                                const long long tok = tok0 + r;
                                if (tok < p.n_tok && col < p.d)
                                    st_global_v4(static_cast<__nv_bfloat16 *>(p.v) + tok * p.d + col, packed);
                                afr[0][mi][hh] = packed.x; afr[0][mi][2 + hh] = packed.y;
                                afr[1][mi][hh] = packed.z; afr[1][mi][2 + hh] = packed.w;
                            }
                        }
#pragma unroll
                        for (int mi = 0; mi < MT; ++mi) {
#pragma unroll
                            for (int ks = 0; ks < 2; ++ks) {
                                const uint32_t blo[2] = {afr[ks][mi][0], afr[ks][mi][2]};      // rows g as B columns
                                const uint32_t bhi[2] = {afr[ks][mi][1], afr[ks][mi][3]};      // rows g + 8
                                mma_bf16(sl[mi], afr[ks][mi], blo);
                                mma_bf16(shh[mi], afr[ks][mi], bhi);
                            }
                        }
                        if (NT > 0) {
#pragma unroll
                            for (int sp = terms - 1; sp >= 0; --sp) {          // small terms first
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt) {
                                    const uint4 b = lds_v4(qbase + sp * kQTerm + (uint32_t)(8 * nt + g) * kWmRow + unit);
                                    const uint32_t b0[2] = {b.x, b.y}, b1[2] = {b.z, b.w};
#pragma unroll
                                    for (int mi = 0; mi < MT; ++mi) {
                                        mma_bf16(part[mi][nt], afr[0][mi], b0);
                                        mma_bf16(part[mi][nt], afr[1][mi], b1);
                                    }
                                }
                            }
                        }
                    }
                    // the chunk's accumulation steps ran in fresh tensor-core accumulators; the running sums are
                    // round-to-nearest fp32 adds
#pragma unroll
                    for (int mi = 0; mi < MT; ++mi) {
                        ss[mi][0] += sl[mi][0]; ss[mi][1] += sl[mi][1]; ss[mi][2] += shh[mi][2]; ss[mi][3] += shh[mi][3];
                    }
                    if (NT > 0) {
#pragma unroll
                        for (int mi = 0; mi < MT; ++mi)
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                                for (int e = 0; e < 4; ++e) acc[mi][nt][e] += part[mi][nt][e];
                    }
                };
                if (active && alive) {
                    if (NT > 0 && (lds_volatile_s32(qlow_a + 8u * qb) | lds_volatile_s32(qlow_a + 8u * qb + 4u)) != 0)
                        chunk_body(std::integral_constant<int, 3>{});
                    else
                        chunk_body(std::integral_constant<int, (NT > 0 ? 1 : 0)>{});
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(empty_a + 8u * st);
                    if (NT > 0) mbar_arrive(qempty_a + 8u * qb);
                }
                if (++st == NS) { st = 0; ph ^= 1u; }
                if (NT > 0) { if (++qb == 2) { qb = 0; qph ^= 1u; } }
            }
            if (active && alive) {
                // key scales: row g's sum of squares is element (g, g) of the rows 0-7 product, held by lane
                // t4 == g / 2 in c0 / c1 by g's parity; row g + 8's is element (g + 8, g) of the rows 8-15 product (c2 / c3)
                if (p.r != nullptr && t4 == (g >> 1)) {
#pragma unroll
                    for (int mi = 0; mi < MT; ++mi) {
                        const float s_lo = (g & 1) ? ss[mi][1] : ss[mi][0], s_hi = (g & 1) ? ss[mi][3] : ss[mi][2];
                        const long long tok = tok0 + row0 + 16 * mi + g;
                        if (tok < p.n_tok) p.r[tok] = rsqrtf(s_lo / (float)p.d + p.eps);
                        if (tok + 8 < p.n_tok) p.r[tok + 8] = rsqrtf(s_hi / (float)p.d + p.eps);
                    }
                }
                if (NT > 0) {
                    // scores: accumulator tiles -> [query][token] through shared memory, then 128-byte rows per query
                    const long long tok = tok0 + row0 + lane;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                        for (int mi = 0; mi < MT; ++mi) {
                            const uint32_t e0 = my_ep + (uint32_t)((2 * t4) * kWmEpPitch + 16 * mi + g) * 4u;
                            sts_f32(e0, acc[mi][nt][0]);
                            sts_f32(e0 + kWmEpPitch * 4u, acc[mi][nt][1]);
                            sts_f32(e0 + 8u * 4u, acc[mi][nt][2]);
                            sts_f32(e0 + (kWmEpPitch + 8u) * 4u, acc[mi][nt][3]);
                        }
                        __syncwarp();
#pragma unroll
                        for (int qq = 0; qq < 8; ++qq) {
                            const int j = 8 * nt + qq;
                            const float val = lds_f32(my_ep + (uint32_t)(qq * kWmEpPitch + lane) * 4u);
                            if (j < nq && lane < RW && tok < p.n_tok) p.dots_s[(long long)(p.j0 + j) * p.dots_qstride + tok] = val;
                        }
                        __syncwarp();
                    }
                }
            }
        }
    } else if (warp == kWmConsumers) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            tma_prefetch_desc(&tmH);
            tma_prefetch_desc(&tmX);
            int st = 0; uint32_t ph = 0;
            int issued = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < p.n_tiles; tile += gridDim.x) {
                const int tok0 = (int)(tile * p.tile_tok);
                for (int c = 0; c < chunks; ++c) {
                    if (!mbar_wait(empty_a + 8u * st, ph ^ 1u, wc, kDevWaitEmpty)) { ok = false; break; }
                    const uint32_t sh = stages_a + (uint32_t)st * stage_bytes, fb = full_a + 8u * st;
                    mbar_arrive_expect_tx(fb, stage_bytes);
                    tma_load_2d(sh, &tmH, fb, c * kWmKC, tok0);
                    tma_load_2d(sh + tile_bytes, &tmX, fb, c * kWmKC, tok0);
                    ++issued;
                    if (++st == NS) { st = 0; ph ^= 1u; }
                }
            }
            if (!ok || lds_volatile_s32(abort_a) != 0) {
                // unwinding (this lane's own wait ran out, or a consumer's did and the consumers stopped waiting for
                // their tiles): let the copies already issued land before the CTA's shared memory is released
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
    } else if (NT > 0) {
        // ------------------------------------------------------------------ query warps
        int qb = 0; uint32_t qph = 0;
        constexpr int kIter = (NT > 0 ? NT : 1) * 8 * (kWmKC / 4) / (32 * kWmQueryWarps);       // float4 per lane and chunk
        const int ql = (warp - kWmConsumers - 1) * 32 + lane;
        for (long long tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x) {
            for (int c = 0; c < chunks; ++c) {
                // all loads of the chunk first (one round trip to L2), rows past nq and columns past d are zero
                float4 q4[kIter];
#pragma unroll
                for (int it = 0; it < kIter; ++it) {
                    const int idx = ql + 32 * kWmQueryWarps * it;
                    const int j = idx >> 4, col = c * kWmKC + 4 * (idx & 15);
                    q4[it] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (j < nq && col < p.d) q4[it] = __ldg(reinterpret_cast<const float4 *>(p.Q + (long long)(p.j0 + j) * p.d + col));
                }
                if (!mbar_wait<true>(qempty_a + 8u * qb, qph ^ 1u, wc, kDevWaitScalarSlot)) return;
                const uint32_t qbase = qs_a + (uint32_t)qb * 3u * kQTerm;
                uint32_t low = 0;
#pragma unroll
                for (int it = 0; it < kIter; ++it) {
                    const int idx = ql + 32 * kWmQueryWarps * it;
                    const int j = idx >> 4, u4 = idx & 15;
                    uint32_t h0, m0, l0, h1, m1, l1, h2, m2, l2, h3, m3, l3;
                    split3(q4[it].x, h0, m0, l0); split3(q4[it].y, h1, m1, l1);
                    split3(q4[it].z, h2, m2, l2); split3(q4[it].w, h3, m3, l3);
                    low |= (m0 | m1 | m2 | m3 | l0 | l1 | l2 | l3) & 0x7fffu;       // a term that is not +-0
                    const uint32_t a = qbase + (uint32_t)j * kWmRow + (uint32_t)((((u4 >> 1) ^ (j & 7)) << 4) + (u4 & 1) * 8);
                    sts_v2(a, h0 | (h1 << 16), h2 | (h3 << 16));
                    sts_v2(a + kQTerm, m0 | (m1 << 16), m2 | (m3 << 16));
                    sts_v2(a + 2u * kQTerm, l0 | (l1 << 16), l2 | (l3 << 16));
                }
                low = __any_sync(0xffffffffu, low != 0u) ? 1u : 0u;
                if (lane == 0) sts_s32(qlow_a + 8u * qb + 4u * (uint32_t)(warp - kWmConsumers - 1), (int)low);
                __syncwarp();
                mbar_arrive(qfull_a + 8u * qb);
                if (++qb == 2) { qb = 0; qph ^= 1u; }
            }
        }
    }
}

template <int NT, int MT>
static cudaError_t launch_wm(const CUtensorMap &tmH, const CUtensorMap &tmX, const WriteMmaParams &p, int grid,
                             size_t smem, cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(write_mma_kernel<NT, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    write_mma_kernel<NT, MT><<<grid, wm_threads(MT), smem, stream>>>(tmH, tmX, p);
    return cudaGetLastError();
}

size_t write_mma_smem_bytes(int nt, int tile_tok, int stages) {
    return 1024 + (size_t)stages * 2 * tile_tok * kWmRow + 6 * (size_t)(nt > 0 ? nt : 1) * 1024 +
           (size_t)16 * 8 * kWmEpPitch * 4 + sizeof(WmBars) + 64;
}

int write_mma_ntiles(int nq) {
    const int need = (nq + 7) / 8;
    const int have[] = {0, 1, 2, 3, 4};
    for (int v : have)
        if (need <= v) return v;
    return -1;
}

cudaError_t launch_write_mma(const CUtensorMap &tmH, const CUtensorMap &tmX, const WriteMmaParams &p, int nt, int mt,
                             int grid, cudaStream_t stream) {
    const size_t smem = write_mma_smem_bytes(nt, p.tile_tok, p.stages);
    switch (nt) {
        case 0: return mt == 1 ? launch_wm<0, 1>(tmH, tmX, p, grid, smem, stream) : launch_wm<0, 2>(tmH, tmX, p, grid, smem, stream);
        case 1: return mt == 1 ? launch_wm<1, 1>(tmH, tmX, p, grid, smem, stream) : launch_wm<1, 2>(tmH, tmX, p, grid, smem, stream);
        case 2: return mt == 1 ? launch_wm<2, 1>(tmH, tmX, p, grid, smem, stream) : launch_wm<2, 2>(tmH, tmX, p, grid, smem, stream);
        case 3: return mt == 1 ? launch_wm<3, 1>(tmH, tmX, p, grid, smem, stream) : launch_wm<3, 2>(tmH, tmX, p, grid, smem, stream);
        case 4: return mt == 1 ? launch_wm<4, 1>(tmH, tmX, p, grid, smem, stream) : launch_wm<4, 2>(tmH, tmX, p, grid, smem, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace lb
