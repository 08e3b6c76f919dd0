// Backward of one read over the stacked updates (sm_100a): the bf16 instantiations of read_bwd_kernel
// (lb_read_bwd_impl.cuh), the entry that picks a storage type and shape, and the small kernels around it.
#include "lb_read_bwd_impl.cuh"

namespace lb {

size_t read_bwd_smem_bytes(int fr, int ncw, int wpt, int stages, int n, int vec, int earlier_steps, int qrow_bytes) {
    size_t stage = (size_t)fr * ncw * kChunkBytes + (size_t)qrow_bytes;
    size_t tables = ((2 * kBwdTables + 1) * bwd_table_floats(n, ncw / wpt) + 8 * bwd_table_floats(earlier_steps, ncw / wpt)) * sizeof(float);
    size_t slots = (size_t)fr * vec * sizeof(float) * ncw * 32;
    size_t qrow = (size_t)fr * wpt * 32 * vec * sizeof(float);       // the query, padded to whole chunks
    return 1024 + stages * stage + ((tables + 15) & ~size_t(15)) + slots + qrow + sizeof(BwdSmemTail) + 64;
}

// SOLO: one warp owns a token's whole row (WPT == 1): no exchange between warps, no named barriers, a one-source-deep
// pipeline; g stays packed in registers (unpacked where it is used) to leave room for 4 fragments per lane.
// MODE 0: the plain backward of a read (lb_read_bwd, lb_read_bwd_final, lb_combine_bwd).
// MODE 1 (STEP): the backward of a whole step (lb_step_bwd): always finalising, the newest update's gradient leaves as
//   the gradients of the block output and input instead of being stored.
// MODE 2 (DEFER): lb_step_bwd_deferred. No gradient stack is read or written: phase 2 forms the finished gradient of the
//   newest update from the upstream-gradient rows g and the per-source scalars that the backward steps before this one
//   left behind (this step leaves its own), and hands it out as in MODE 1.
cudaError_t launch_read_bwd(int dtype, int fr, int ncw, const CUtensorMap &tmV, const CUtensorMap &tmG,
                            const CUtensorMap &tmDV, const CUtensorMap &tmH0, const ReadBwdParams &p, int grid,
                            cudaStream_t stream) {
    if (dtype == LB_DTYPE_BF16) return launch_read_bwd_typed<__nv_bfloat16>(fr, ncw, tmV, tmG, tmDV, tmH0, p, grid, stream);
    return launch_read_bwd_f32(fr, ncw, tmV, tmG, tmDV, tmH0, p, grid, stream);
}

// dq[c] = scale * sum_rows dq_part[row][c]; fixed summation order (deterministic).
// Replaces the torch reduction of the per-program partials (fused_dattn.py:785).
__global__ void __launch_bounds__(256) dq_reduce_kernel(const float *__restrict__ part, int rows, float *__restrict__ dq,
                                                        int d, float scale) {
    __shared__ float red[8][33];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + cx;
    float s = 0.f;
    if (col < d)
        for (int r = ry; r < rows; r += 8) s += part[(long long)r * d + col];
    red[ry][cx] = s;
    __syncthreads();
    if (ry == 0 && col < d) {
        float tsum = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) tsum += red[k][cx];
        dq[col] = tsum * scale;
    }
}

// Qp[j][chunk][e4][lane][0..3] = Q[j][chunk * BW + lane * VEC + 4 e4 + 0..3] (zero past d): the order in which the
// lanes of the deferred backward read a query row from shared memory.
__global__ void __launch_bounds__(256) permute_queries_kernel(const float *__restrict__ Q, float *__restrict__ Qp, int nq, int d,
                                                              int vec, int row_floats) {
    const int bw = 32 * vec, v4 = vec / 4;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < (long long)nq * row_floats;
         idx += (long long)gridDim.x * blockDim.x) {
        const int j = (int)(idx / row_floats), o = (int)(idx - (long long)j * row_floats);
        const int chunk = o / bw, r = o - chunk * bw;          // r = (e4 * 32 + lane) * 4 + c
        const int e4 = r / 128, lane = (r >> 2) & 31, c = r & 3;
        const int col = chunk * bw + lane * vec + 4 * e4 + c;
        Qp[idx] = (e4 < v4 && col < d) ? Q[(long long)j * d + col] : 0.f;
    }
}

cudaError_t launch_permute_queries(const float *Q, float *Qp, int nq, int d, int vec, int row_floats, cudaStream_t stream) {
    const long long total = (long long)nq * row_floats;
    if (total == 0) return cudaSuccess;
    permute_queries_kernel<<<(unsigned)((total + 255) / 256 < 1024 ? (total + 255) / 256 : 1024), 256, 0, stream>>>(Q, Qp, nq, d, vec, row_floats);
    return cudaGetLastError();
}

cudaError_t launch_dq_reduce(const float *dq_part, int rows, float *dq, int d, float scale, cudaStream_t stream) {
    dq_reduce_kernel<<<(d + 31) / 32, 256, 0, stream>>>(dq_part, rows, dq, d, scale);
    return cudaGetLastError();
}

}  // namespace lb
