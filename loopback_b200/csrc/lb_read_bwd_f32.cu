// Backward of one read over the stacked updates (sm_100a): the fp32 instantiations of read_bwd_kernel
// (lb_read_bwd_impl.cuh), in a translation unit of their own so that they compile beside the bf16 ones.
#include "lb_read_bwd_impl.cuh"

namespace lb {

cudaError_t launch_read_bwd_f32(int fr, int ncw, const CUtensorMap &tmV, const CUtensorMap &tmG, const CUtensorMap &tmDV,
                                const CUtensorMap &tmH0, const ReadBwdParams &p, int grid, cudaStream_t stream) {
    return launch_read_bwd_typed<float>(fr, ncw, tmV, tmG, tmDV, tmH0, p, grid, stream);
}

}  // namespace lb
