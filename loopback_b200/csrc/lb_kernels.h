// Internal interface between the C-ABI layer (lb_api.cu) and the kernel translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#define LB_DTYPE_F32 0
#define LB_DTYPE_BF16 1

namespace lb {

struct ReadFwdParams {
    const float *R;        // [N][n_tok] key scales
    const float *dots;     // [N][n_tok] the scores of this read's query (row block of DOTS, or a scratch row block)
    const float *cbar;     // [n_tok][n] installed coefficients (used when tc_prev is null)
    const float *tc_prev;  // [n_tok][n-1] the previous read's coefficients, or null: cbar = lam * (tc_prev, 1)
    float lam;             // decay applied with tc_prev (1 inside an iteration, 1 - beta at its end)
    int blend;             // 1: base = proposal + beta (h0 - proposal) formed in the kernel (tmBase = proposal)
    float beta;
    const float *c0;       // [n] the read's prior
    void *out;             // [n_tok][d]
    float *TC;             // [n_tok][n]
    float *LG;             // [n_tok][n] logits, or null (no backward)
    float *LSE;            // [n_tok] or null
    float *LSE0;           // [n_tok] or null
    long long n_tok;
    int d;
    int n;
    int chunks;            // ceil(d * elem / 512)
    int wpt;               // consumer warps per token; tokens per tile = consumer warps / wpt
    int col_groups;        // ceil(chunks / (FR * wpt))
    long long tok_tiles;   // ceil(n_tok / tokens per tile)
    int rank4;             // 1: one 4-D TMA box per stage (d a multiple of the chunk width), 0: one box per chunk
    int stages;
    int sps;               // sources per stage (1..4; > 1 only with rank4)
    float inv_sqrt_d;
    int *err_word;         // device error word (see lb_device_error)
    long long wait_cycles; // limit of every bounded wait
    int test_skip_item;    // test hook: CTA 0's producer leaves out its k-th tile copy (0 = off), so that a consumer's
                           // bounded wait runs out and the unwinding path executes
};

size_t read_fwd_smem_bytes(int fr, int ncw, int stages, int sps);
cudaError_t launch_read_fwd(int dtype, int fr, int ncw, const CUtensorMap &tmV, const CUtensorMap &tmBase,
                            const CUtensorMap &tmH0, const ReadFwdParams &p, int grid, cudaStream_t stream);
cudaError_t launch_scores(int dtype, const void *V, const float *q, float *dots, long long n_tok, int d, int n,
                          int sms, cudaStream_t stream);

struct WriteParams {
    const void *h;         // [n_tok][d]
    const void *x;         // [n_tok][d]
    void *v;               // [n_tok][d]  (slice s of the stack)
    float *r;              // [n_tok]     (slice s of R), may be null
    const float *Q;        // [NQ][d] fp32 queries, or null (no scores)
    float *dots_s;         // DOTS + s * n_tok: element (j, t) at dots_s[j * N * n_tok + t]
    long long n_tok;
    long long dots_qstride;   // N * n_tok
    int d;
    int j0;                // first query whose read sees this update
    int nq;                // queries j0 .. j0 + nq - 1 are scored
    float eps;
    int write_tt;          // tokens per lane (1 or 2); 0 = choose by size
};

cudaError_t launch_write(int dtype, const WriteParams &p, int sms, cudaStream_t stream);

// The tensor-core write (bf16 rows, training-sized batches): tiles of tile_tok tokens (a multiple of 32, <= 256)
struct WriteMmaParams : WriteParams {
    int tile_tok;
    int chunks;            // 64-column chunks per row
    int stages;            // TMA ring depth (2..4)
    long long n_tiles;
    int *err_word;
    long long wait_cycles;
};
int write_mma_ntiles(int nq);                                   // query tiles of 8 the kernel is built for, or -1
size_t write_mma_smem_bytes(int nt, int tile_tok, int stages);
cudaError_t launch_write_mma(const CUtensorMap &tmH, const CUtensorMap &tmX, const WriteMmaParams &p, int nt, int mt,
                             int grid, cudaStream_t stream);   // mt: 16-token tiles per consumer warp (1 or 2)
cudaError_t launch_rstd_fwd(int dtype, const void *x, float *r, long long n_tok, int d, float eps, int sms,
                            cudaStream_t stream);
// mode 0: gx = gr (-r^3/d) x written;  mode 1: gx += round(gr (-r^3/d) x), rounded to the storage type
cudaError_t launch_rstd_bwd(int dtype, const void *x, const float *r, const float *gr, void *gx, long long n_tok,
                            int d, int mode, int sms, cudaStream_t stream);
cudaError_t launch_neg(int dtype, const void *g, void *out, long long n_elem, int sms, cudaStream_t stream);
// acc = round(beta g) (accumulate == 0) or round(acc + round(beta g)), storage-type arithmetic
cudaError_t launch_scale_acc(int dtype, const void *g, void *acc, float beta, int accumulate, long long n_elem, int sms,
                             cudaStream_t stream);

// One whole forward step for decode-sized batches (lb_step_fwd): one CTA per token, ct column threads x sg source groups
struct StepSmallParams {
    const void *h, *x, *h0;   // [n_tok][d]; h0 only when blend
    void *V;                  // [N][n_tok][d]: slice n-1 is written, slices below are read
    float *R;                 // [N][n_tok]
    const float *q;           // [d] the read's query (row n-2 of the queries)
    const float *tc_prev;     // [n_tok][n-1]
    const float *c0;          // [n]
    void *out;                // [n_tok][d]
    float *TC, *LG, *LSE, *LSE0;
    long long n_tok;
    int d, n;
    float lam, beta, eps, inv_sqrt_d;
    int blend;
    int ct, sg;
};
size_t step_small_smem_bytes(int ct, int sg, int vec);
cudaError_t launch_step_small(int dtype, const StepSmallParams &p, cudaStream_t stream);

struct ReadBwdParams {
    const float *R;        // [N][n_tok]
    float *dR;             // [N][n_tok]
    void *dV;              // [N][n_tok][d] (stores go here; loads of the old value come through TMA)
    const float *q;        // [d] fp32
    const float *gt;       // [n_tok][n] or null
    const float *cbar;     // [n_tok][n] (used when tc_prev is null)
    const float *tc_prev;  // [n_tok][n-1] or null: cbar = lam * (tc_prev, 1) and dcbar receives d/d tc_prev [n_tok][n-1]
    float lam;
    const float *c0;       // [n]
    const float *LSE;      // [n_tok]
    const float *LSE0;     // [n_tok]
    const float *LG;       // [n_tok][n]
    float *dcbar;          // [n_tok][n]
    float *dq_part;        // [grid][d] scratch: one partial row per CTA
    long long n_tok;
    long long tok_tiles;
    int d;
    int n;
    int chunks;
    int wpt;               // warps per token (a power of two); tokens per tile = consumer warps / wpt
    int rank4;             // as in ReadFwdParams
    int stages;
    int accum;             // 0: dV / dR are written; 1: added into
    int finalize;          // 1: also add the key-scale gradient term of source n-1 into dV[n-1] (its last reader)
    void *neg_out;         // [n_tok][d] or null: receives -dV[n-1] when finalize is set
    // the step's own gradients, with finalize (one autograd node for the write and the read of update n-1):
    void *dh_out;          // [n_tok][d] or null: dV[n-1] + the gradient of the read's base with respect to the block output
    void *dh0;             // [n_tok][d] or null: receives (dh0_accum: is added) round(beta g), the blend's h0 gradient
    int dh0_accum;
    int blend;             // 1: the read closed an iteration (base = h + beta (h0 - h))
    float beta;
    int skip_final_store;  // 1: dV[n-1] itself is not stored (nothing reads it after its last reader)
    long long wait_cycles; // limit of every bounded wait
    float inv_sqrt_d;
    int *err_word;
    // the deferred form (lb_step_bwd_deferred); Gst == null selects the forms above
    void *Gst = nullptr;          // [N][n_tok][d]: the g row of every backward step (slice n-1 is written, slices n.. are read)
    float *Wt = nullptr;          // [N][N][n_tok]: entry [s][i] = step s's coefficient of g in the gradient of update i < s
    float *KQt = nullptr;         // ... and of the step's query q_s
    const float *Qall = nullptr;  // [N-1][chunks * 512 / elem] every query, permuted by lb_permute_queries
    int qrow_bytes = 0;           // bytes of such a row: a query row travels with each g tile
    int n_total = 0;              // N
    int fin2 = 0;                 // 1 (the step-1 backward): also finish update 0 into dv0_out / neg0_out
    void *dv0_out = nullptr, *neg0_out = nullptr;
};

size_t read_bwd_smem_bytes(int fr, int ncw, int wpt, int stages, int n, int vec, int earlier_steps = 0, int qrow_bytes = 0);
cudaError_t launch_read_bwd(int dtype, int fr, int ncw, const CUtensorMap &tmV, const CUtensorMap &tmG,
                            const CUtensorMap &tmDV, const CUtensorMap &tmH0, const ReadBwdParams &p, int grid,
                            cudaStream_t stream);
cudaError_t launch_permute_queries(const float *Q, float *Qp, int nq, int d, int vec, int row_floats, cudaStream_t stream);
cudaError_t launch_dq_reduce(const float *dq_part, int rows, float *dq, int d, float scale, cudaStream_t stream);

// The one-shot all-reduce of the query gradient through peer memory (lb_peer_allreduce)
constexpr int kMaxPeers = 16;      // ranks of a node
constexpr int kPeerCtas = 32;      // CTAs (= slices of the buffer) at most
// a rank's flag block, in 32-bit words: [2 phases][kMaxPeers source ranks][kPeerCtas], then the CTAs' call counters
constexpr int kPeerFlagWords = 2 * kMaxPeers * kPeerCtas + kPeerCtas;
struct PeerReduceParams {
    const float *bufs[kMaxPeers];  // every rank's buffer, rank-ordered (bufs[rank] is this rank's own)
    unsigned *flags[kMaxPeers];    // every rank's flag block
    float *out;                    // [4 n4] the sum
    long long n4;                  // 16-byte groups of the buffer
    long long slice4;              // groups per CTA (filled in by the launcher)
    int rank, world;
    long long wait_cycles;
    int *err_word;
};
int peer_allreduce_ctas(long long n4);
cudaError_t launch_peer_allreduce(PeerReduceParams p, cudaStream_t stream);

}  // namespace lb
