// C-ABI layer: argument checks, tile-shape selection, TMA descriptors, launches. See include/loopback_b200.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include <cudaTypedefs.h>

#include "../../include/loopback_b200.h"
#include "lb_common.cuh"
#include "lb_kernels.h"

// one error word per device: the first bounded wait of any kernel that runs out records its code here
__device__ int g_lb_device_error = 0;

namespace {

constexpr int kMaxGrid = 304;                 // rows of the query-gradient scratch (>= 2 CTAs per SM on 148 SMs)
constexpr size_t kMaxSmem = 227 * 1024;

thread_local std::string t_err;

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    t_err = buf;
    return code;
}

int cuda_fail(cudaError_t e, const char *what) {
    return fail(LB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

struct Options {
    int fwd_stages = 0, bwd_stages = 0, fwd_fr = 0, grid_cap = 0, fwd_warps = 0, bwd_warps = 0, bwd_wpt = 0,
        tma_per_chunk = 0, write_tt = 0, write_mt = 0, fwd_sps = 0, write_tile = 0, write_stages = 0, wait_cycles = 0, test_skip_item = 0;
} g_opt;

struct DeviceInfo {
    int sms = 0;
    int cc_major = 0;
    int *err_word = nullptr;
    bool ok = false;
};

int device_info(DeviceInfo *out) {
    static std::mutex mu;
    static DeviceInfo cache[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(LB_ERR_CUDA, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lk(mu);
    if (!cache[dev].ok) {
        DeviceInfo di;
        if ((e = cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
            return cuda_fail(e, "cudaDeviceGetAttribute(sm count)");
        if ((e = cudaDeviceGetAttribute(&di.cc_major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
            return cuda_fail(e, "cudaDeviceGetAttribute(cc major)");
        if (di.cc_major != 10)
            return fail(LB_ERR_CUDA, "device %d has compute capability %d.x; this library is built for sm_100a only",
                        dev, di.cc_major);
        if ((e = cudaGetSymbolAddress(reinterpret_cast<void **>(&di.err_word), g_lb_device_error)) != cudaSuccess)
            return cuda_fail(e, "cudaGetSymbolAddress(device error word)");
        di.ok = true;
        cache[dev] = di;
    }
    *out = cache[dev];
    return LB_OK;
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    });
    return fn;
}

// A tiled descriptor over [outer][n_tok][d] (outer == 0: no outer dimension).
//   box_chunks == 0: dimensions (d, n_tok[, outer]), box = 512 bytes x box_tok tokens: one chunk of every token;
//   box_chunks  > 0: the row is split into whole 512-byte chunks, dimensions (chunk width, chunks, n_tok[, outer]),
//                    box = 512 bytes x box_chunks chunks x box_tok tokens: a whole tile in one copy, token-major.
//                    Needs d to be a multiple of the chunk width.
int make_map(CUtensorMap *m, const void *base, int dtype, long long n_tok, int d, int outer, int box_tok,
             int box_chunks, int box_outer = 1) {
    auto fn = encode_fn();
    if (!fn) return fail(LB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const int elem = dtype == LB_DTYPE_BF16 ? 2 : 4;
    const cuuint64_t bw = lb::kChunkBytes / elem;
    cuuint64_t dims[4];
    cuuint64_t strides[3];
    cuuint32_t box[4];
    cuuint32_t estr[4] = {1, 1, 1, 1};
    cuuint32_t rank = 0;
    if (box_chunks > 0) {
        dims[0] = bw; dims[1] = (cuuint64_t)d / bw; dims[2] = (cuuint64_t)n_tok;
        strides[0] = lb::kChunkBytes; strides[1] = (cuuint64_t)d * elem;
        box[0] = (cuuint32_t)bw; box[1] = (cuuint32_t)box_chunks; box[2] = (cuuint32_t)box_tok;
        rank = 3;
    } else {
        dims[0] = (cuuint64_t)d; dims[1] = (cuuint64_t)n_tok;
        strides[0] = (cuuint64_t)d * elem;
        box[0] = (cuuint32_t)bw; box[1] = (cuuint32_t)box_tok;
        rank = 2;
    }
    if (outer > 0) {
        dims[rank] = (cuuint64_t)outer;
        strides[rank - 1] = (cuuint64_t)d * elem * (cuuint64_t)n_tok;
        box[rank] = (cuuint32_t)box_outer;
        ++rank;
    }
    CUresult r = fn(m, dtype == LB_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                    rank, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return LB_OK;
}

// h / x of the tensor-core write: 2-D, boxes of box_tok rows x 64 bf16 columns, 128-byte swizzle
int make_map_sw128(CUtensorMap *m, const void *base, long long n_tok, int d, int box_tok) {
    auto fn = encode_fn();
    if (!fn) return fail(LB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)n_tok};
    cuuint64_t strides[1] = {(cuuint64_t)d * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_tok};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return LB_OK;
}

long long wait_limit() { return g_opt.wait_cycles > 0 ? (long long)g_opt.wait_cycles : lb::kWaitCycles; }

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_common(long long n_tok, int d, int dtype) {
    if (dtype != LB_DTYPE_BF16 && dtype != LB_DTYPE_F32) return fail(LB_ERR_ARG, "dtype %d is neither LB_DTYPE_F32 nor LB_DTYPE_BF16", dtype);
    if (n_tok < 0 || d <= 0) return fail(LB_ERR_ARG, "n_tok=%lld, d=%d: sizes must be positive", n_tok, d);
    if (n_tok >= (1LL << 31)) return fail(LB_ERR_UNSUPPORTED, "n_tok=%lld does not fit the 32-bit TMA coordinates", n_tok);
    const long long row = (long long)d * (dtype == LB_DTYPE_BF16 ? 2 : 4);
    if (row % 16 != 0) return fail(LB_ERR_ALIGN, "row size %lld bytes (d=%d) is not a multiple of 16", row, d);
    if (row > 32 * lb::kChunkBytes) return fail(LB_ERR_UNSUPPORTED, "row size %lld bytes exceeds the supported 16384", row);
    return LB_OK;
}

int chunks_of(int d, int dtype) {
    const int row = d * (dtype == LB_DTYPE_BF16 ? 2 : 4);
    return (row + lb::kChunkBytes - 1) / lb::kChunkBytes;
}

}  // namespace

// sets the calling thread's error message from another translation unit of this library (not exported)
extern "C" int lb_fail_message(int code, const char *msg) { return fail(code, "%s", msg); }

#pragma GCC visibility push(default)
extern "C" {

int lb_version(void) { return LB_VERSION; }

const char *lb_last_error_string(void) { return t_err.c_str(); }

int lb_device_error(int clear) {
    int v = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
    e = cudaMemcpyFromSymbol(&v, g_lb_device_error, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyFromSymbol(device error word)");
    if (clear && v != 0) {
        int z = 0;
        e = cudaMemcpyToSymbol(g_lb_device_error, &z, sizeof(int));
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyToSymbol(device error word)");
    }
    if (v != 0) fail(LB_ERR_DEVICE, "a kernel gave up a bounded wait (code %d)", v);
    return v;
}

int lb_set_option(const char *name, int value) {
    if (!name) return fail(LB_ERR_ARG, "option name is NULL");
    if (!strcmp(name, "reset_all")) g_opt = Options();
    else if (!strcmp(name, "fwd_stages")) g_opt.fwd_stages = value;
    else if (!strcmp(name, "bwd_stages")) g_opt.bwd_stages = value;
    else if (!strcmp(name, "fwd_fr")) g_opt.fwd_fr = value;
    else if (!strcmp(name, "grid_cap")) g_opt.grid_cap = value;
    else if (!strcmp(name, "fwd_warps")) g_opt.fwd_warps = value;
    else if (!strcmp(name, "bwd_warps")) g_opt.bwd_warps = value;
    else if (!strcmp(name, "bwd_wpt")) g_opt.bwd_wpt = value;
    else if (!strcmp(name, "tma_per_chunk")) g_opt.tma_per_chunk = value;
    else if (!strcmp(name, "write_tt")) g_opt.write_tt = value;
    else if (!strcmp(name, "write_mt")) g_opt.write_mt = value;
    else if (!strcmp(name, "fwd_sps")) g_opt.fwd_sps = value;
    else if (!strcmp(name, "write_tile")) g_opt.write_tile = value;
    else if (!strcmp(name, "write_stages")) g_opt.write_stages = value;
    else if (!strcmp(name, "wait_cycles")) g_opt.wait_cycles = value;
    else if (!strcmp(name, "test_skip_item")) g_opt.test_skip_item = value;
    else return fail(LB_ERR_ARG, "unknown option '%s'", name);
    return LB_OK;
}

int lb_write(const void *h, const void *x, void *V, float *R, const float *Q, float *DOTS, int64_t n_tok, int d, int N,
             int NQ, int s, float eps, int dtype, void *stream) {
    int rc = check_common(n_tok, d, dtype);
    if (rc) return rc;
    if (!h || !x || !V) return fail(LB_ERR_ARG, "lb_write: h, x and V must be non-NULL");
    if (N <= 0 || s < 0 || s >= N) return fail(LB_ERR_ARG, "lb_write: step %d outside [0, %d)", s, N);
    if (!R) Q = nullptr;                       // without R only V[s] is written: Q is ignored
    if (Q && (!DOTS || NQ < 0 || NQ > N)) return fail(LB_ERR_ARG, "lb_write: scores need DOTS and 0 <= NQ <= N");
    if (!aligned16(h) || !aligned16(x) || !aligned16(V) || (Q && !aligned16(Q)))
        return fail(LB_ERR_ALIGN, "lb_write: h, x, V and Q must be 16-byte aligned");
    DeviceInfo di;
    if ((rc = device_info(&di))) return rc;
    const long long elem = dtype == LB_DTYPE_BF16 ? 2 : 4;
    lb::WriteParams p;
    p.h = h; p.x = x;
    p.v = static_cast<char *>(V) + (long long)s * n_tok * d * elem;
    p.r = R ? R + (long long)s * n_tok : nullptr;
    p.Q = (Q && R) ? Q : nullptr;
    p.j0 = s > 0 ? s - 1 : 0;
    p.nq = p.Q ? NQ - p.j0 : 0;
    if (p.nq <= 0) { p.nq = 0; p.Q = nullptr; }
    p.dots_s = DOTS ? DOTS + (long long)s * n_tok : nullptr;
    p.dots_qstride = (long long)N * n_tok;
    p.n_tok = n_tok; p.d = d; p.eps = eps; p.write_tt = g_opt.write_tt == 1 || g_opt.write_tt == 2 ? g_opt.write_tt : 0;
    // bf16 rows in training-sized batches (every SM gets at least 32 tokens): the persistent tensor-core kernel
    const int nt = lb::write_mma_ntiles(p.nq);
    if (dtype == LB_DTYPE_BF16 && d >= 64 && nt >= 0 && n_tok > 0 &&
        (g_opt.write_tt == 3 || (g_opt.write_tt == 0 && n_tok >= 32LL * di.sms))) {
        const long long blocks32 = (n_tok + 31) / 32;
        const long long rounds = (blocks32 + 8LL * di.sms - 1) / (8LL * di.sms);
        const long long per = (blocks32 + di.sms * rounds - 1) / (di.sms * rounds);        // 1..8
        lb::WriteMmaParams mp;
        static_cast<lb::WriteParams &>(mp) = p;
        mp.tile_tok = (int)per * 32;
        if (g_opt.write_tile >= 32 && g_opt.write_tile <= 256 && g_opt.write_tile % 32 == 0) mp.tile_tok = g_opt.write_tile;
        mp.chunks = (d + 63) / 64;
        mp.n_tiles = (n_tok + mp.tile_tok - 1) / mp.tile_tok;
        mp.err_word = di.err_word;
        mp.wait_cycles = wait_limit();
        mp.stages = g_opt.write_stages >= 2 && g_opt.write_stages <= 8 ? g_opt.write_stages : 4;
        while (mp.stages > 2 && lb::write_mma_smem_bytes(nt, mp.tile_tok, mp.stages) > 227 * 1024) --mp.stages;
        CUtensorMap tmH, tmX;
        if ((rc = make_map_sw128(&tmH, h, n_tok, d, mp.tile_tok))) return rc;
        if ((rc = make_map_sw128(&tmX, x, n_tok, d, mp.tile_tok))) return rc;
        const int grid = (int)(mp.n_tiles < di.sms ? mp.n_tiles : di.sms);
        cudaError_t e = lb::launch_write_mma(tmH, tmX, mp, nt, g_opt.write_mt == 1 ? 1 : 2, grid, static_cast<cudaStream_t>(stream));
        return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_write launch");
    }
    cudaError_t e = lb::launch_write(dtype, p, di.sms, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_write launch");
}

int lb_write_bwd_dx(const void *g, void *dx, int64_t n_elem, int dtype, void *stream) {
    if (dtype != LB_DTYPE_BF16 && dtype != LB_DTYPE_F32) return fail(LB_ERR_ARG, "bad dtype %d", dtype);
    if (!g || !dx || n_elem < 0) return fail(LB_ERR_ARG, "lb_write_bwd_dx: NULL pointer or negative size");
    if (!aligned16(g) || !aligned16(dx) || (n_elem * (dtype == LB_DTYPE_BF16 ? 2 : 4)) % 16)
        return fail(LB_ERR_ALIGN, "lb_write_bwd_dx: pointers and byte size must be multiples of 16");
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc) return rc;
    cudaError_t e = lb::launch_neg(dtype, g, dx, n_elem, di.sms, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_write_bwd_dx launch");
}

int lb_rstd_fwd(const void *x, float *r, int64_t n_tok, int d, float eps, int dtype, void *stream) {
    int rc = check_common(n_tok, d, dtype);
    if (rc) return rc;
    if (!x || !r) return fail(LB_ERR_ARG, "lb_rstd_fwd: NULL pointer");
    if (!aligned16(x)) return fail(LB_ERR_ALIGN, "lb_rstd_fwd: x must be 16-byte aligned");
    DeviceInfo di;
    if ((rc = device_info(&di))) return rc;
    cudaError_t e = lb::launch_rstd_fwd(dtype, x, r, n_tok, d, eps, di.sms, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_rstd_fwd launch");
}

static int rstd_bwd_common(const void *x, const float *r, const float *gr, void *gx, int64_t n_tok, int d, int dtype,
                           int mode, void *stream) {
    int rc = check_common(n_tok, d, dtype);
    if (rc) return rc;
    if (!x || !r || !gr || !gx) return fail(LB_ERR_ARG, "lb_rstd_bwd: NULL pointer");
    if (!aligned16(x) || !aligned16(gx)) return fail(LB_ERR_ALIGN, "lb_rstd_bwd: x and gx must be 16-byte aligned");
    DeviceInfo di;
    if ((rc = device_info(&di))) return rc;
    cudaError_t e = lb::launch_rstd_bwd(dtype, x, r, gr, gx, n_tok, d, mode, di.sms, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_rstd_bwd launch");
}

int lb_rstd_bwd(const void *x, const float *r, const float *gr, void *gx, int64_t n_tok, int d, int dtype, void *stream) {
    return rstd_bwd_common(x, r, gr, gx, n_tok, d, dtype, 0, stream);
}

int lb_rstd_bwd_acc(const void *x, const float *r, const float *gr, void *dv, int64_t n_tok, int d, int dtype,
                    void *stream) {
    return rstd_bwd_common(x, r, gr, dv, n_tok, d, dtype, 1, stream);
}

int lb_scores(const void *V, const float *q, float *dots, int64_t n_tok, int d, int N, int n, int dtype, void *stream) {
    int rc = check_common(n_tok, d, dtype);
    if (rc) return rc;
    if (!V || !q || !dots) return fail(LB_ERR_ARG, "lb_scores: NULL pointer");
    if (n < 1 || n > N) return fail(LB_ERR_ARG, "lb_scores: n=%d outside [1, N=%d]", n, N);
    if (!aligned16(V) || !aligned16(q)) return fail(LB_ERR_ALIGN, "lb_scores: V and q must be 16-byte aligned");
    DeviceInfo di;
    if ((rc = device_info(&di))) return rc;
    cudaError_t e = lb::launch_scores(dtype, V, q, dots, n_tok, d, n, di.sms, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_scores launch");
}

static int read_fwd_impl(const void *V, const float *R, const float *DOTS, int qi, const void *base, const void *h0,
                         float beta, const float *cbar, const float *tc_prev, float lam, const float *c0, void *out,
                         float *TC, float *LG, float *LSE, float *LSE0, int64_t n_tok, int d, int N, int n, int dtype,
                         void *stream);

int lb_read_fwd(const void *V, const float *R, const float *DOTS, int qi, const void *base, const float *cbar,
                const float *c0, void *out, float *TC, float *LG, float *LSE, float *LSE0, int64_t n_tok, int d, int N,
                int n, int dtype, void *stream) {
    if (!cbar) return fail(LB_ERR_ARG, "lb_read_fwd: NULL pointer");
    return read_fwd_impl(V, R, DOTS, qi, base, nullptr, 0.f, cbar, nullptr, 1.f, c0, out, TC, LG, LSE, LSE0, n_tok, d, N, n,
                         dtype, stream);
}

int lb_combine_fwd(const void *V, const float *R, const float *DOTS, int qi, const void *proposal, const void *h0,
                   float beta, const float *tc_prev, float lam, const float *c0, void *out, float *TC, float *LG,
                   float *LSE, float *LSE0, int64_t n_tok, int d, int N, int n, int dtype, void *stream) {
    if (n < 2 || !tc_prev) return fail(LB_ERR_ARG, "lb_combine_fwd: needs n >= 2 and the previous read's coefficients");
    if (h0 && !aligned16(h0)) return fail(LB_ERR_ALIGN, "lb_combine_fwd: h0 must be 16-byte aligned");
    return read_fwd_impl(V, R, DOTS, qi, proposal, h0, beta, nullptr, tc_prev, lam, c0, out, TC, LG, LSE, LSE0, n_tok, d,
                         N, n, dtype, stream);
}

static int read_fwd_impl(const void *V, const float *R, const float *DOTS, int qi, const void *base, const void *h0,
                         float beta, const float *cbar, const float *tc_prev, float lam, const float *c0, void *out,
                         float *TC, float *LG, float *LSE, float *LSE0, int64_t n_tok, int d, int N, int n, int dtype,
                         void *stream) {
    int rc = check_common(n_tok, d, dtype);
    if (rc) return rc;
    if (!V || !R || !DOTS || !base || (!cbar && !tc_prev) || !c0 || !out || !TC) return fail(LB_ERR_ARG, "lb_read_fwd: NULL pointer");
    if ((LG != nullptr) != (LSE != nullptr) || (LG != nullptr) != (LSE0 != nullptr))
        return fail(LB_ERR_ARG, "lb_read_fwd: LG, LSE and LSE0 must be given together");
    if (n < 1 || n > N) return fail(LB_ERR_ARG, "lb_read_fwd: n=%d outside [1, N=%d]", n, N);
    if (n > LB_MAX_SOURCES) return fail(LB_ERR_UNSUPPORTED, "lb_read_fwd: n=%d exceeds LB_MAX_SOURCES=%d", n, LB_MAX_SOURCES);
    if (qi < 0) return fail(LB_ERR_ARG, "lb_read_fwd: query row %d is negative", qi);
    if (!aligned16(V) || !aligned16(base) || !aligned16(out))
        return fail(LB_ERR_ALIGN, "lb_read_fwd: V, base and out must be 16-byte aligned");
    if (n_tok == 0) return LB_OK;
    DeviceInfo di;
    if ((rc = device_info(&di))) return rc;

    const int nch = chunks_of(d, dtype);
    const int elem = dtype == LB_DTYPE_BF16 ? 2 : 4;
    const bool rank4 = !g_opt.tma_per_chunk && (d * elem) % lb::kChunkBytes == 0;
    // Tile shape: consumer warps (16, 12 or 8), warps per token and fragments per warp. A tile normally spans the
    // whole row (one column group); the choice avoids idle fragments first, then prefers stages near 16 KiB.
    // With too few tokens to give every SM a tile, the row is cut into column groups instead (8-token tiles).
    int ncw = 0, wpt = 0, fr = 0, best_cost = 1 << 30;
    static const int kNcw[3] = {8, 12, 16};
    for (int a = 0; a < 3; ++a) {
        if (g_opt.fwd_warps && g_opt.fwd_warps != kNcw[a]) continue;
        for (int w = 1; w <= kNcw[a]; ++w) {
            if (kNcw[a] % w) continue;
            const int f = (nch + w - 1) / w;
            if (f > 4 || (g_opt.fwd_fr && g_opt.fwd_fr != f)) continue;
            const int stage_kb = nch * (kNcw[a] / w) / 2;
            const int off = stage_kb > 16 ? stage_kb - 16 : 16 - stage_kb;
            const int cost = (f * w - nch) * 64 + off * 2 + a;
            if (cost < best_cost) { best_cost = cost; ncw = kNcw[a]; wpt = w; fr = f; }
        }
    }
    if (ncw == 0) return fail(LB_ERR_UNSUPPORTED, "lb_read_fwd: no tile shape covers d=%d (row of %d chunks)", d, nch);
    int bt = ncw / wpt;
    long long tok_tiles = (n_tok + bt - 1) / bt;
    int cg = 1;
    if (tok_tiles < di.sms) {            // few tokens: 8 tokens x (fr chunks) tiles, as many column groups as it takes
        ncw = 8; wpt = 1; bt = 8;
        tok_tiles = (n_tok + 7) / 8;
        fr = nch < 4 ? nch : 4;
        while (fr > 1 && tok_tiles * ((nch + fr - 1) / fr) < di.sms) --fr;
        cg = (nch + fr - 1) / fr;
    }
    // ring depth: 6 stages of a full-size (12-16 KiB) tile measured best (8 and more cost 2-4 %: more requests in
    // flight than the memory system orders well); small tiles (decode-sized batches) get a deeper ring so that a CTA
    // still keeps ~128 KiB in flight
    // Small tiles also take several sources per stage (one TMA box over the source axis): the hand-shake of a stage
    // costs about as much for 4 KiB as for 16 KiB, and a decode-sized read is made of nothing else.
    const int tile_bytes = fr * ncw * lb::kChunkBytes;
    int sps = 1;
    if (rank4 && n >= 4) sps = tile_bytes <= 4 * 1024 ? 4 : (tile_bytes <= 8 * 1024 ? 2 : 1);
    if (rank4 && g_opt.fwd_sps >= 1 && g_opt.fwd_sps <= 4) sps = g_opt.fwd_sps;
    const int stage_bytes = sps * tile_bytes;
    int stages = g_opt.fwd_stages > 0 ? g_opt.fwd_stages : 6;
    if (g_opt.fwd_stages <= 0 && stage_bytes < 12 * 1024) stages = 128 * 1024 / stage_bytes;
    if (stages > 32) stages = 32;
    while (stages > 2 && lb::read_fwd_smem_bytes(fr, ncw, stages, sps) > kMaxSmem) --stages;

    CUtensorMap tmV, tmB, tmH;
    if ((rc = make_map(&tmV, V, dtype, n_tok, d, N, bt, rank4 ? fr * wpt : 0, sps))) return rc;
    if ((rc = make_map(&tmB, base, dtype, n_tok, d, 0, bt, rank4 ? fr * wpt : 0))) return rc;
    if ((rc = make_map(&tmH, h0 ? h0 : base, dtype, n_tok, d, 0, bt, rank4 ? fr * wpt : 0))) return rc;

    lb::ReadFwdParams p;
    p.R = R;
    p.dots = DOTS + (long long)qi * N * n_tok;
    p.cbar = cbar; p.tc_prev = tc_prev; p.lam = lam; p.blend = h0 ? 1 : 0; p.beta = beta;
    p.c0 = c0; p.out = out; p.TC = TC; p.LG = LG; p.LSE = LSE; p.LSE0 = LSE0;
    p.n_tok = n_tok; p.d = d; p.n = n; p.chunks = nch; p.wpt = wpt; p.col_groups = cg; p.tok_tiles = tok_tiles;
    p.stages = stages; p.sps = sps;
    p.rank4 = rank4 ? 1 : 0;
    p.inv_sqrt_d = 1.0f / sqrtf((float)d);
    p.err_word = di.err_word;
    p.wait_cycles = wait_limit(); p.test_skip_item = g_opt.test_skip_item;
    const long long tiles = tok_tiles * cg;
    int cap = g_opt.grid_cap > 0 ? g_opt.grid_cap : di.sms;
    if (cap > kMaxGrid) cap = kMaxGrid;
    const int grid = (int)(tiles < cap ? tiles : cap);
    cudaError_t e = lb::launch_read_fwd(dtype, fr, ncw, tmV, tmB, tmH, p, grid, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_read_fwd launch");
}

int lb_step_fwd(const void *h, const void *x, const void *h0, float beta, void *V, float *R, const float *Q,
                const float *tc_prev, float lam, const float *c0, void *out, float *TC, float *LG, float *LSE, float *LSE0,
                int64_t n_tok, int d, int N, int s, float eps, int dtype, void *stream) {
    int rc = check_common(n_tok, d, dtype);
    if (rc) return rc;
    if (!h || !x || !V || !R || !Q || !tc_prev || !c0 || !out || !TC) return fail(LB_ERR_ARG, "lb_step_fwd: NULL pointer");
    if ((LG != nullptr) != (LSE != nullptr) || (LG != nullptr) != (LSE0 != nullptr))
        return fail(LB_ERR_ARG, "lb_step_fwd: LG, LSE and LSE0 must be given together");
    if (s < 1 || s >= N) return fail(LB_ERR_ARG, "lb_step_fwd: step %d outside [1, N=%d)", s, N);
    if (s + 1 > LB_MAX_SOURCES) return fail(LB_ERR_UNSUPPORTED, "lb_step_fwd: %d sources exceed LB_MAX_SOURCES=%d", s + 1, LB_MAX_SOURCES);
    if (!aligned16(h) || !aligned16(x) || !aligned16(V) || !aligned16(out) || !aligned16(Q) || (h0 && !aligned16(h0)))
        return fail(LB_ERR_ALIGN, "lb_step_fwd: h, x, h0, V, out and Q must be 16-byte aligned");
    if (((long long)d * 4) % 16) return fail(LB_ERR_ALIGN, "lb_step_fwd: the query rows must be multiples of 16 bytes");
    if (n_tok > 65535LL * 16) return fail(LB_ERR_UNSUPPORTED, "lb_step_fwd: meant for decode-sized batches; %lld tokens is not one", (long long)n_tok);
    if (n_tok == 0) return LB_OK;
    DeviceInfo di;
    if ((rc = device_info(&di))) return rc;
    const int elem = dtype == LB_DTYPE_BF16 ? 2 : 4;
    lb::StepSmallParams p;
    p.h = h; p.x = x; p.h0 = h0; p.V = V; p.R = R; p.q = Q + (long long)(s - 1) * d; p.tc_prev = tc_prev; p.c0 = c0;
    p.out = out; p.TC = TC; p.LG = LG; p.LSE = LSE; p.LSE0 = LSE0;
    p.n_tok = n_tok; p.d = d; p.n = s + 1; p.lam = lam; p.beta = beta; p.eps = eps; p.inv_sqrt_d = 1.0f / sqrtf((float)d);
    p.blend = h0 ? 1 : 0;
    const int frags = (d * elem + 15) / 16;
    p.ct = (frags + 31) / 32 * 32;
    p.sg = p.ct >= 1024 ? 1 : (1024 / p.ct > 4 ? 4 : 1024 / p.ct);
    if (lb::step_small_smem_bytes(p.ct, p.sg, 16 / elem) > kMaxSmem) return fail(LB_ERR_UNSUPPORTED, "lb_step_fwd: row too wide");
    cudaError_t e = lb::launch_step_small(dtype, p, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_step_fwd launch");
}

size_t lb_read_bwd_scratch_bytes(int d) { return d > 0 ? (size_t)kMaxGrid * (size_t)d * sizeof(float) : 0; }

// what a finalising backward hands out beyond dV / dR when the write and the read of update n-1 are one autograd node
struct StepGrads {
    void *dh = nullptr;        // gradient of the block output
    void *dh0 = nullptr;       // gradient of the loop input (an iteration's last read only)
    int dh0_accum = 0;
    int blend = 0;
    float beta = 0.f;
    int skip_final_store = 0;
    // the deferred form (G != null): no gradient stack; `dV` of read_bwd_impl is then the g stack
    float *Wt = nullptr, *KQt = nullptr;
    const float *Qall = nullptr;
    int deferred = 0;
    void *dv0 = nullptr, *dx0 = nullptr;
};

static int read_bwd_impl(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g,
                         const float *gt, const float *cbar, const float *tc_prev, float lam, const float *c0,
                         const float *LG, const float *LSE, const float *LSE0, float *dcbar, float *dq, void *scratch,
                         int64_t n_tok, int d, int N, int n, int accum, int finalize, void *neg_out, int dtype,
                         void *stream, const StepGrads &sg = StepGrads());

int lb_read_bwd(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g, const float *gt,
                const float *cbar, const float *c0, const float *LG, const float *LSE, const float *LSE0, float *dcbar,
                float *dq, void *scratch, int64_t n_tok, int d, int N, int n, int accum, int dtype, void *stream) {
    if (!cbar) return fail(LB_ERR_ARG, "lb_read_bwd: NULL pointer");
    return read_bwd_impl(V, R, dV, dR, q, g, gt, cbar, nullptr, 1.f, c0, LG, LSE, LSE0, dcbar, dq, scratch, n_tok, d, N, n,
                         accum, 0, nullptr, dtype, stream);
}

int lb_combine_bwd(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g, const float *gt,
                   const float *tc_prev, float lam, const float *c0, const float *LG, const float *LSE,
                   const float *LSE0, float *dtc_prev, float *dq, void *scratch, void *neg_out, int finalize,
                   int64_t n_tok, int d, int N, int n, int accum, int dtype, void *stream) {
    if (n < 2 || !tc_prev) return fail(LB_ERR_ARG, "lb_combine_bwd: needs n >= 2 and the previous read's coefficients");
    if (neg_out && !aligned16(neg_out)) return fail(LB_ERR_ALIGN, "lb_combine_bwd: neg_out must be 16-byte aligned");
    return read_bwd_impl(V, R, dV, dR, q, g, gt, nullptr, tc_prev, lam, c0, LG, LSE, LSE0, dtc_prev, dq, scratch, n_tok, d,
                         N, n, accum, finalize, neg_out, dtype, stream);
}

int lb_read_bwd_final(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g,
                      const float *gt, const float *cbar, const float *c0, const float *LG, const float *LSE,
                      const float *LSE0, float *dcbar, float *dq, void *scratch, void *neg_out, int64_t n_tok, int d,
                      int N, int n, int accum, int dtype, void *stream) {
    if (neg_out && !aligned16(neg_out)) return fail(LB_ERR_ALIGN, "lb_read_bwd_final: neg_out must be 16-byte aligned");
    if (!cbar) return fail(LB_ERR_ARG, "lb_read_bwd_final: NULL pointer");
    return read_bwd_impl(V, R, dV, dR, q, g, gt, cbar, nullptr, 1.f, c0, LG, LSE, LSE0, dcbar, dq, scratch, n_tok, d, N, n,
                         accum, 1, neg_out, dtype, stream);
}

int lb_step_bwd(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g, const float *gt,
                const float *tc_prev, float lam, const float *c0, const float *LG, const float *LSE, const float *LSE0,
                float *dtc_prev, float *dq, void *scratch, void *dh, void *dx, void *dh0, int dh0_accum, int blend,
                float beta, int64_t n_tok, int d, int N, int n, int accum, int dtype, void *stream) {
    if (n < 2 || !tc_prev) return fail(LB_ERR_ARG, "lb_step_bwd: needs n >= 2 and the previous read's coefficients");
    if (!dh || !dx) return fail(LB_ERR_ARG, "lb_step_bwd: dh and dx must be non-NULL");
    if (!aligned16(dh) || !aligned16(dx) || (dh0 && !aligned16(dh0)))
        return fail(LB_ERR_ALIGN, "lb_step_bwd: dh, dx and dh0 must be 16-byte aligned");
    if (dh0 && !blend) return fail(LB_ERR_ARG, "lb_step_bwd: dh0 is only produced by a read that closes an iteration");
    StepGrads sg;
    sg.dh = dh; sg.dh0 = dh0; sg.dh0_accum = dh0 ? dh0_accum : 0; sg.blend = blend ? 1 : 0; sg.beta = beta;
    sg.skip_final_store = 1;
    return read_bwd_impl(V, R, dV, dR, q, g, gt, nullptr, tc_prev, lam, c0, LG, LSE, LSE0, dtc_prev, dq, scratch, n_tok, d,
                         N, n, accum, 1, dx, dtype, stream, sg);
}

size_t lb_permuted_query_row_floats(int d, int dtype) {
    if (d <= 0 || (dtype != LB_DTYPE_BF16 && dtype != LB_DTYPE_F32)) return 0;
    return (size_t)chunks_of(d, dtype) * (lb::kChunkBytes / (dtype == LB_DTYPE_BF16 ? 2 : 4));
}

int lb_permute_queries(const float *Q, float *Qp, int NQ, int d, int dtype, void *stream) {
    int rc = check_common(0, d, dtype);
    if (rc) return rc;
    if (!Q || !Qp || NQ < 0) return fail(LB_ERR_ARG, "lb_permute_queries: NULL pointer or negative size");
    cudaError_t e = lb::launch_permute_queries(Q, Qp, NQ, d, dtype == LB_DTYPE_BF16 ? 8 : 4,
                                               (int)lb_permuted_query_row_floats(d, dtype), static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_permute_queries launch");
}

int lb_peer_flag_words(void) { return lb::kPeerFlagWords; }

int lb_peer_allreduce(const float *const *bufs, unsigned int *const *flags, int rank, int world, float *out, int64_t n,
                      void *stream) {
    if (!bufs || !flags || !out) return fail(LB_ERR_ARG, "lb_peer_allreduce: NULL pointer");
    if (world < 1 || world > lb::kMaxPeers || rank < 0 || rank >= world)
        return fail(LB_ERR_ARG, "lb_peer_allreduce: needs 1 <= world <= LB_MAX_PEERS and 0 <= rank < world");
    if (n < 0 || n % 4) return fail(LB_ERR_ARG, "lb_peer_allreduce: n must be a non-negative multiple of 4 floats");
    if (n == 0) return LB_OK;
    lb::PeerReduceParams p{};
    for (int r = 0; r < world; ++r) {
        if (!bufs[r] || !flags[r]) return fail(LB_ERR_ARG, "lb_peer_allreduce: NULL peer pointer");
        if (!aligned16(bufs[r]) || ((uintptr_t)flags[r] & 3u)) return fail(LB_ERR_ALIGN, "lb_peer_allreduce: buffers must be 16-byte aligned");
        p.bufs[r] = bufs[r]; p.flags[r] = flags[r];
    }
    if (!aligned16(out)) return fail(LB_ERR_ALIGN, "lb_peer_allreduce: out must be 16-byte aligned");
    DeviceInfo di;
    int rc;
    if ((rc = device_info(&di))) return rc;
    p.out = out; p.n4 = n / 4; p.rank = rank; p.world = world;
    p.wait_cycles = wait_limit(); p.err_word = di.err_word;
    cudaError_t e = lb::launch_peer_allreduce(p, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_peer_allreduce launch");
}

int lb_step_bwd_deferred(const void *V, const float *R, void *G, float *dR, float *Wt, float *KQt, const float *Q,
                         const float *Qp, const void *g, const float *gt, const float *tc_prev, float lam, const float *c0, const float *LG,
                         const float *LSE, const float *LSE0, float *dtc_prev, float *dq, void *scratch, void *dh, void *dx,
                         void *dh0, int dh0_accum, int blend, float beta, void *dv0, void *dx0, int64_t n_tok, int d, int N,
                         int n, int first, int dtype, void *stream) {
    if (n < 2 || !tc_prev) return fail(LB_ERR_ARG, "lb_step_bwd_deferred: needs n >= 2 and the previous read's coefficients");
    if (!G || !Wt || !KQt || !Q || !Qp || !dh || !dx) return fail(LB_ERR_ARG, "lb_step_bwd_deferred: NULL pointer");
    if (!aligned16(G) || !aligned16(Q) || !aligned16(Qp) || !aligned16(dh) || !aligned16(dx) || (dh0 && !aligned16(dh0)) ||
        (dv0 && !aligned16(dv0)) || (dx0 && !aligned16(dx0)))
        return fail(LB_ERR_ALIGN, "lb_step_bwd_deferred: G, Q, dh, dx, dh0, dv0 and dx0 must be 16-byte aligned");
    if (((long long)d * 4) % 16) return fail(LB_ERR_ALIGN, "lb_step_bwd_deferred: the query rows must be multiples of 16 bytes");
    if (dh0 && !blend) return fail(LB_ERR_ARG, "lb_step_bwd_deferred: dh0 is only produced by a read that closes an iteration");
    if ((dv0 != nullptr) != (dx0 != nullptr) || (dv0 && n != 2))
        return fail(LB_ERR_ARG, "lb_step_bwd_deferred: dv0 and dx0 come together, from the step-1 backward (n == 2) only");
    StepGrads sg;
    sg.dh = dh; sg.dh0 = dh0; sg.dh0_accum = dh0 ? dh0_accum : 0; sg.blend = blend ? 1 : 0; sg.beta = beta;
    sg.skip_final_store = 1;
    sg.deferred = 1; sg.Wt = Wt; sg.KQt = KQt; sg.Qall = Qp; sg.dv0 = dv0; sg.dx0 = dx0;
    return read_bwd_impl(V, R, G, dR, Q + (long long)(n - 2) * d, g, gt, nullptr, tc_prev, lam, c0, LG, LSE, LSE0, dtc_prev, dq,
                         scratch, n_tok, d, N, n, first ? 0 : 1, 1, dx, dtype, stream, sg);
}

static int read_bwd_impl(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g,
                         const float *gt, const float *cbar, const float *tc_prev, float lam, const float *c0,
                         const float *LG, const float *LSE, const float *LSE0, float *dcbar, float *dq, void *scratch,
                         int64_t n_tok, int d, int N, int n, int accum, int finalize, void *neg_out, int dtype,
                         void *stream, const StepGrads &sg) {
    int rc = check_common(n_tok, d, dtype);
    if (rc) return rc;
    if (!V || !R || !dV || !dR || !q || !g || (!cbar && !tc_prev) || !c0 || !LG || !LSE || !LSE0 || !dcbar || !dq || !scratch)
        return fail(LB_ERR_ARG, "lb_read_bwd: NULL pointer");
    if (n < 1 || n > N) return fail(LB_ERR_ARG, "lb_read_bwd: n=%d outside [1, N=%d]", n, N);
    if (n > LB_MAX_SOURCES) return fail(LB_ERR_UNSUPPORTED, "lb_read_bwd: n=%d exceeds LB_MAX_SOURCES=%d", n, LB_MAX_SOURCES);
    if (!aligned16(V) || !aligned16(dV) || !aligned16(g) || !aligned16(q) || !aligned16(scratch))
        return fail(LB_ERR_ALIGN, "lb_read_bwd: V, dV, g, q and scratch must be 16-byte aligned");
    DeviceInfo di;
    if ((rc = device_info(&di))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n_tok == 0) {
        cudaError_t e0 = cudaMemsetAsync(dq, 0, sizeof(float) * d, st);
        return e0 == cudaSuccess ? LB_OK : cuda_fail(e0, "cudaMemsetAsync(dq)");
    }

    const int nch = chunks_of(d, dtype);
    const int elem = dtype == LB_DTYPE_BF16 ? 2 : 4;
    const bool rank4 = !g_opt.tma_per_chunk && (d * elem) % lb::kChunkBytes == 0;
    // Tile shape. A row of at most 4 chunks goes to ONE warp per token (8 consumer warps, 8 tokens per tile): no
    // exchange between warps and the most work per barrier wait. Wider rows are split over several warps per token:
    // consumer warps (12, 16 or 8), warps per token and fragments per warp are chosen for no idle fragments first,
    // then tiles of at least 12 KiB, then 2 fragments per warp.
    int ncw = 0, wpt = 0, fr = 0, best_cost = 1 << 30;
    static const int kNcw[3] = {12, 16, 8}, kFrMax[3] = {2, 2, 4};
    if (nch <= 4 && g_opt.bwd_wpt <= 1 && (g_opt.bwd_warps == 0 || g_opt.bwd_warps == 8 || g_opt.bwd_warps == 4)) {
        // 8 consumer warps and one CTA per SM, or ("bwd_warps" = 4) half-size CTAs of 4 consumer warps, two per SM:
        // two independent pipelines whose phases drift apart (no faster since phase 1 became straight-line code: an option only)
        const bool half = g_opt.bwd_warps == 4;
        ncw = half ? 4 : 8; wpt = 1; fr = nch;
    } else if (sg.deferred && !g_opt.bwd_warps && !g_opt.bwd_wpt && (nch == 8 || nch == 16 || nch == 32)) {
        // the deferred form keeps g packed and has registers for 3 or 4 fragments per warp: 8 consumer warps, fewer warps
        // per token to exchange partial dot products between (measured: -15 % at 8 chunks, -6 % at 12)
        ncw = 8; fr = 4; wpt = nch / 4;
    } else if (sg.deferred && !g_opt.bwd_warps && !g_opt.bwd_wpt && (nch == 6 || nch == 12 || nch == 24)) {
        ncw = 8; fr = 3; wpt = nch / 3;
    } else {
        for (int a = 0; a < 3; ++a) {
            if (g_opt.bwd_warps && g_opt.bwd_warps != kNcw[a]) continue;
            for (int w = 2; w <= kNcw[a]; ++w) {
                if (kNcw[a] % w || kNcw[a] / w > 8) continue;     // named barriers 1..8: one per token of the tile
                if (g_opt.bwd_wpt && g_opt.bwd_wpt != w) continue;
                const int f = (nch + w - 1) / w;
                if (f > kFrMax[a]) continue;
                const int stage = nch * (kNcw[a] / w) * lb::kChunkBytes;
                const int cost = (f * w - nch) * 64 + (stage < 12 * 1024 ? 16 : 0) + (f == 2 ? 0 : (f == 3 ? 2 : (f == 1 ? 3 : 4))) * 2 + a;
                if (cost < best_cost) { best_cost = cost; ncw = kNcw[a]; wpt = w; fr = f; }
            }
        }
    }
    if (ncw == 0) return fail(LB_ERR_UNSUPPORTED, "lb_read_bwd: no tile shape covers d=%d (row of %d chunks)", d, nch);
    const int bt = ncw / wpt;
    const int vec = dtype == LB_DTYPE_BF16 ? 8 : 4;
    int stages = g_opt.bwd_stages > 0 ? g_opt.bwd_stages : 8;
    if (stages > 12) stages = 12;
    const int earlier = sg.deferred ? N - n : 0, qrow = sg.deferred ? (int)lb_permuted_query_row_floats(d, dtype) * 4 : 0;
    const size_t smem_cap = ncw == 4 ? (kMaxSmem - 2048) / 2 : kMaxSmem;      // two half-size CTAs share an SM
    while (stages > 2 && lb::read_bwd_smem_bytes(fr, ncw, wpt, stages, n, vec, earlier, qrow) > smem_cap) --stages;
    if (lb::read_bwd_smem_bytes(fr, ncw, wpt, stages, n, vec, earlier, qrow) > smem_cap)
        return fail(LB_ERR_UNSUPPORTED, "lb_read_bwd: shared memory does not fit for d=%d, n=%d", d, n);

    CUtensorMap tmV, tmG, tmDV, tmH0;
    if ((rc = make_map(&tmV, V, dtype, n_tok, d, N, bt, rank4 ? nch : 0))) return rc;
    if ((rc = make_map(&tmG, g, dtype, n_tok, d, 0, bt, rank4 ? nch : 0))) return rc;
    if ((rc = make_map(&tmDV, dV, dtype, n_tok, d, N, bt, rank4 ? nch : 0))) return rc;
    if ((rc = make_map(&tmH0, sg.dh0 ? sg.dh0 : g, dtype, n_tok, d, 0, bt, rank4 ? nch : 0))) return rc;

    lb::ReadBwdParams p;
    p.R = R; p.dR = dR; p.dV = dV; p.q = q; p.gt = gt; p.cbar = cbar; p.tc_prev = tc_prev; p.lam = lam; p.c0 = c0; p.LSE = LSE; p.LSE0 = LSE0; p.LG = LG;
    p.dcbar = dcbar; p.dq_part = static_cast<float *>(scratch);
    p.n_tok = n_tok; p.tok_tiles = (n_tok + bt - 1) / bt; p.d = d; p.n = n; p.chunks = nch; p.wpt = wpt;
    p.stages = stages; p.rank4 = rank4 ? 1 : 0; p.accum = accum ? 1 : 0; p.finalize = finalize ? 1 : 0;
    p.neg_out = finalize ? neg_out : nullptr; p.inv_sqrt_d = 1.0f / sqrtf((float)d);
    p.dh_out = finalize ? sg.dh : nullptr; p.dh0 = finalize ? sg.dh0 : nullptr; p.dh0_accum = sg.dh0_accum;
    p.blend = sg.blend; p.beta = sg.beta; p.skip_final_store = finalize ? sg.skip_final_store : 0;
    p.err_word = di.err_word; p.wait_cycles = wait_limit();
    if (sg.deferred) {
        p.Gst = dV; p.Wt = sg.Wt; p.KQt = sg.KQt; p.Qall = sg.Qall; p.qrow_bytes = qrow; p.n_total = N;
        p.fin2 = sg.dv0 ? 1 : 0; p.dv0_out = sg.dv0; p.neg0_out = sg.dx0;
    }
    int cap = g_opt.grid_cap > 0 ? g_opt.grid_cap : di.sms * (ncw == 4 ? 2 : 1);
    if (cap > kMaxGrid) cap = kMaxGrid;
    const int grid = (int)(p.tok_tiles < cap ? p.tok_tiles : cap);
    cudaError_t e = lb::launch_read_bwd(dtype, fr, ncw, tmV, tmG, tmDV, tmH0, p, grid, st);
    if (e != cudaSuccess) return cuda_fail(e, "lb_read_bwd launch");
    if (p.dh0 != nullptr && wpt > 1) {
        // shapes with several warps per token leave the loop input's gradient to a small kernel of its own (in their
        // main kernel the extra code cost every launch 2-3 %, boundary read or not)
        e = lb::launch_scale_acc(dtype, g, p.dh0, p.beta, p.dh0_accum, (long long)n_tok * d, di.sms, st);
        if (e != cudaSuccess) return cuda_fail(e, "lb_step_bwd h0-gradient launch");
    }
    e = lb::launch_dq_reduce(p.dq_part, grid, dq, d, p.inv_sqrt_d, st);
    return e == cudaSuccess ? LB_OK : cuda_fail(e, "lb_read_bwd dq reduction launch");
}

}  // extern "C"
#pragma GCC visibility pop
