// Shared device/host helpers of the Loopback read kernels (sm_100a).
//
// Data model used by every kernel in this directory
//   * a "row" is one token's d elements; rows are cut into CHUNKS of 512 bytes (256 bf16 / 128 fp32 columns);
//   * a FRAGMENT is 16 bytes of a chunk (8 bf16 / 4 fp32); lane l of a warp owns fragment l of a chunk, so one
//     warp instruction touches one whole 512-byte chunk row (conflict-free in shared memory, coalesced in HBM);
//   * streaming kernels stage TILES of BT tokens x NCHT chunks in shared memory with TMA
//     (cp.async.bulk.tensor, no multicast), laid out [chunk][token][512 B].
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lb {

constexpr int kChunkBytes = 512;          // one TMA box row
constexpr int kMaxSources = 128;          // n (= sources of a read) the shared-memory scalar tables are sized for

// ---------------------------------------------------------------------------------------------------------
// device-side error word: kernels never trap or spin forever; a wait that runs out records where and returns.
// ---------------------------------------------------------------------------------------------------------
enum DeviceError : int {
    kDevOk = 0,
    kDevWaitFull = 1,      // a consumer gave up waiting for a TMA tile
    kDevWaitEmpty = 2,     // the producer gave up waiting for a free stage
    kDevWaitScalars = 3,   // a consumer gave up waiting for the scalar tables of a tile
    kDevWaitScalarSlot = 4,
    kDevWaitDrain = 5,     // the producer gave up waiting for its own copies in flight at exit
    kDevWaitPeer = 6,      // the peer all-reduce gave up waiting for another rank's flag
};

// The error word itself is a __device__ int owned by lb_api.cu (one per device); kernels get its address.

// ---------------------------------------------------------------------------------------------------------
// PTX wrappers: mbarrier + TMA
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// All shared-memory traffic of the streaming kernels goes through 32-bit shared-window addresses (smem_u32 of the
// dynamic shared memory base, plus offsets): the loads are real ld.shared instructions and no 64-bit generic
// pointer has to stay live in registers.
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ int lds_volatile_s32(uint32_t a) {
    int v;
    asm volatile("ld.volatile.shared.s32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}
__device__ __forceinline__ void sts_s32(uint32_t a, int v) {
    asm volatile("st.shared.s32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_f4(uint32_t a, const float4 &v) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// Bounded wait. The abort flag lives in shared memory: the first wait of a CTA that runs out sets it (and the
// device error word), every later wait of that CTA then fails at once, so a stuck CTA unwinds in one time-out.
constexpr long long kWaitCycles = 4000000000LL;   // the default limit: ~2 s at B200 clocks

struct WaitCtx {
    uint32_t abort_flag;        // shared-window address of the CTA's abort flag
    int *err_word;              // global memory, per device
    long long limit;            // cycles a wait may take (kWaitCycles unless the "wait_cycles" option says otherwise)
};

// `relaxed` waits (the scalar warps': they run a tile ahead of the consumers) sleep between polls, so
// that their polling does not take issue slots from the consumer warps on the same scheduler.
template <bool kRelaxed = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx &wc, int what) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (kRelaxed) __nanosleep(128);
        if ((++spins & 255u) == 0u) {
            if (lds_volatile_s32(wc.abort_flag)) return false;
            if (clock64() - t0 > wc.limit) {
                sts_s32(wc.abort_flag, what);
                atomicCAS(wc.err_word, 0, what);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on an mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---------------------------------------------------------------------------------------------------------
// storage types: a fragment is one uint4 (16 B) holding VEC elements
// ---------------------------------------------------------------------------------------------------------
template <typename T> struct Store;

template <> struct Store<__nv_bfloat16> {
    static constexpr int kVec = 8;
    static constexpr int kBytes = 2;
    static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    // bf16 -> fp32 is a shift: exact
    __device__ __forceinline__ static void unpack(const uint4 &u, float (&f)[8]) {
        f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
        f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
        f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xffff0000u);
        f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xffff0000u);
    }
    __device__ __forceinline__ static uint32_t pack2(float lo, float hi) {
        __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);      // round-to-nearest-even, .x = lo
        return *reinterpret_cast<uint32_t *>(&b);
    }
    __device__ __forceinline__ static uint4 pack(const float (&f)[8]) {
        return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
    }
    // the value a store of `x` would hold, back in fp32
    __device__ __forceinline__ static float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

    // the same fragment as element PAIRS, the operand shape of the packed fp32 instructions (fma.rn.f32x2)
    static constexpr int kPairs = 4;
    __device__ __forceinline__ static float2 unpack1(uint32_t u) {
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
    }
    __device__ __forceinline__ static void unpack2(const uint4 &u, float2 (&f)[4]) {
        f[0] = unpack1(u.x); f[1] = unpack1(u.y); f[2] = unpack1(u.z); f[3] = unpack1(u.w);
    }
    __device__ __forceinline__ static uint4 pack2v(const float2 (&f)[4]) {
        return make_uint4(pack2(f[0].x, f[0].y), pack2(f[1].x, f[1].y), pack2(f[2].x, f[2].y), pack2(f[3].x, f[3].y));
    }
    // round(prev + round(o)) per element: o is rounded to bf16, then one native bf16 add (exact sum, one rounding)
    __device__ __forceinline__ static uint32_t hadd(uint32_t a, uint32_t b) {
        __nv_bfloat162 r = __hadd2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    }
    __device__ __forceinline__ static uint4 accum(const uint4 &prev, const float2 (&o)[4]) {
        const uint4 r = pack2v(o);
        return make_uint4(hadd(prev.x, r.x), hadd(prev.y, r.y), hadd(prev.z, r.z), hadd(prev.w, r.w));
    }
    __device__ __forceinline__ static uint4 negate(const uint4 &u) {
        return make_uint4(u.x ^ 0x80008000u, u.y ^ 0x80008000u, u.z ^ 0x80008000u, u.w ^ 0x80008000u);
    }
};

template <> struct Store<float> {
    static constexpr int kVec = 4;
    static constexpr int kBytes = 4;
    static constexpr CUtensorMapDataType kTma = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    __device__ __forceinline__ static void unpack(const uint4 &u, float (&f)[4]) {
        f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
    }
    __device__ __forceinline__ static uint4 pack(const float (&f)[4]) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                          __float_as_uint(f[3]));
    }
    __device__ __forceinline__ static float round(float x) { return x; }

    static constexpr int kPairs = 2;
    __device__ __forceinline__ static void unpack2(const uint4 &u, float2 (&f)[2]) {
        f[0] = make_float2(__uint_as_float(u.x), __uint_as_float(u.y));
        f[1] = make_float2(__uint_as_float(u.z), __uint_as_float(u.w));
    }
    __device__ __forceinline__ static uint4 pack2v(const float2 (&f)[2]) {
        return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y), __float_as_uint(f[1].x),
                          __float_as_uint(f[1].y));
    }
    __device__ __forceinline__ static uint4 accum(const uint4 &prev, const float2 (&o)[2]) {
        float2 pf[2];
        unpack2(prev, pf);
        pf[0] = __fadd2_rn(pf[0], o[0]);
        pf[1] = __fadd2_rn(pf[1], o[1]);
        return pack2v(pf);
    }
    __device__ __forceinline__ static uint4 negate(const uint4 &u) {
        return make_uint4(u.x ^ 0x80000000u, u.y ^ 0x80000000u, u.z ^ 0x80000000u, u.w ^ 0x80000000u);
    }
};

// acc += a.lo * b.lo (acc0) and a.hi * b.hi (acc1) for two packed bf16 pairs: the mixed-precision fma of sm_100
// (bf16 x bf16 product, exact in fp32, added in fp32 with one rounding) -- the same values as unpacking both operands to
// fp32 and an fp32 fma, without the unpacking
__device__ __forceinline__ void fma_bf16x2(uint32_t a, uint32_t b, float &acc0, float &acc1) {
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t"
        "mov.b32 {al, ah}, %2;\n\t"
        "mov.b32 {bl, bh}, %3;\n\t"
        "fma.rn.f32.bf16 %0, al, bl, %0;\n\t"
        "fma.rn.f32.bf16 %1, ah, bh, %1;\n\t}"
        : "+f"(acc0), "+f"(acc1)
        : "r"(a), "r"(b));
}

// streaming global accesses: read-once data bypasses L1, stores do not allocate in L1
__device__ __forceinline__ uint4 ld_global_stream_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void st_global_v4(void *p, const uint4 &v) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// reductions inside aligned groups of `width` lanes (width a power of two <= 32)
__device__ __forceinline__ float group_sum(float v, int width) {
    for (int o = width >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float group_max(float v, int width) {
    for (int o = width >> 1; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace lb
