// Launchers of the block step's CUDA kernels (sm_100a).  Every pointer is device memory.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ava {

// ---- launches with programmatic dependent launch -----------------------------------------------------------------
// Every kernel of the step starts with pdl_enter(): it lets the next kernel in the stream be scheduled early
// (griddepcontrol.launch_dependents) and then waits until the kernel before it has completed and its writes are
// visible (griddepcontrol.wait), so the order of the work is that of plain stream launches while launch latency and
// block scheduling overlap the tail of the kernel before.  Without the launch attribute both instructions do nothing.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_enter() {
#ifdef AVA_PDL_EARLY_TRIGGER
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

extern thread_local cudaError_t g_launch_error;
extern int g_pdl;  // 1: launch with the programmatic-serialization attribute (the default)

// Every kernel asks for the same split of an SM's on-chip memory between shared memory and L1.  An SM cannot change the
// split while blocks are resident on it, so kernels that ask for different splits do not run side by side on one SM: a
// kernel of another stream then waits until the SM has drained, however much room is left (measured: a lane's RMS norm
// waited 116 us for another lane's state pass to end).  With one preference for all, a lane's small kernels start beside
// another lane's state pass.  A kernel that needs more than the preferred share still gets it.  percent_for_this >= 0
// (given before the kernel's first launch) asks for another split for that kernel: the tensor-core kernels of prompt
// reading, which run alone on their stream, take all of it so that two of their blocks share an SM.
void prefer_max_shared(const void* kernel, int percent_for_this = -1);

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    prefer_max_shared(reinterpret_cast<const void*>(kernel));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 1 : 0;
    const cudaError_t rc = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (rc != cudaSuccess && g_launch_error == cudaSuccess) g_launch_error = rc;  // kept until take_launch_error reads it
    return rc;
}
// The first launch that was refused on this thread since the last call (cudaSuccess: none), and forgets it.  The step
// asks after queueing its kernels, so a refused launch (a grid too large, a kernel image that did not load) fails the
// call instead of leaving a result that lacks one kernel's work.
inline cudaError_t take_launch_error() {
    const cudaError_t rc = g_launch_error;
    g_launch_error = cudaSuccess;
    return rc;
}

// Status word in device memory that kernels OR bits into; the host reads it when it reads the step's results.
enum : uint32_t {
    ST_NONFINITE = 1u,     // a gate, key or value of the fast-weight memory was not finite
    ST_WAIT_TIMEOUT = 2u,  // a bounded wait on a copy barrier ran out
    ST_ENGRAM_FULL = 4u,   // the engram store had no room for this token
    ST_BAD_TOKEN = 8u,     // a token id outside the vocabulary
};

// ---- int8-weight products -----------------------------------------------------------------------------------
enum GemmEpilogue { EPI_STORE = 0, EPI_ADD = 1, EPI_LIF = 2 };

// The --neuromod signals of a step lie as [rows][NM_STRIDE] floats (NE, ACh, DA, one unused).
constexpr int NM_STRIDE = 4;

struct LifParams {
    const float* beta;   // [d] leak (already sigmoid of the parameter)
    const float* theta;  // [d] or nullptr (1.0)
    const float* rho;    // [d] or nullptr: no adaptive threshold
    const float* gain;   // [d] or nullptr
    float* v;            // [M, d] membranes, updated in place
    float* s;            // [M, d] spikes, updated in place (this step's spikes are what W_out reads)
    float* a;            // [M, d] adaptation trace or nullptr
    const float* ne;     // --neuromod NE: the current (after lif_scale) times ne[row * NM_STRIDE], or nullptr
    int spikes;          // 0 binary, 1 ternary, 2 int2
    int lif_scale;       // current times (1 - beta)
};

// The product kernels take this struct by value.  It is kept at 128 bytes (pointers first, no padding): with a larger
// parameter block the compiler gave the 64x64 tile kernel 80 registers instead of 64, three resident blocks per SM
// instead of four, and the widest product of the step lost 7%.
struct GemmArgs {
    const float* A;      // [M, K] activations, row stride lda
    const int8_t* W;     // [K, N] int8 weights, row stride ldw
    const float* scale;  // [N]
    float* C;            // [M, N] output (EPI_STORE / EPI_ADD), row stride ldc
    int lda, ldw, ldc;
    int M, N, K;
    LifParams lif;       // EPI_LIF (N == d).  EPI_ADD reads only lif.ne: when not null, the product's row r is multiplied
                         // by lif.ne[r * NM_STRIDE] before the add (--neuromod DA on the MLP's output)
};
static_assert(sizeof(GemmArgs) == 128, "parameter block of the product kernels");

// What a product for a few rows does to its input rows in shared memory before the chains start, instead of a kernel of
// its own in front of it (one sequence talking is bound by the count of kernels, not by their work):
//   PRO_RMS   the block's RMS norm: x (mean(x^2) + eps)^-1/2 gain (src/model/fstep.rs:212-220)
//   PRO_POST  the memory's head norm and silu output gate (src/model/fstep/arch.rs:842-852)
// Every block of the product takes the row's ordered sum itself, while its strip of weights is on the way.
enum GemvPrologue { PRO_NONE = 0, PRO_RMS = 1, PRO_POST = 2 };
struct GemvPro {
    int kind = PRO_NONE;
    const float* gain = nullptr;   // PRO_RMS: [K]
    const float* gate = nullptr;   // PRO_POST: the output gate's pre-activation [M, ldg], or nullptr
    int ldg = 0;
    int hs = 0;                    // PRO_POST: head size (K is a multiple)
    float* out = nullptr;          // not null: the rows after the prologue [M, K], written by the first block of columns
};

// C = A . W with f32 activations, int8 weights, one fused multiply-add per term in the order k = 0, 1, ... from +0,
// the sum then times scale[n]: the bits of the reference's int8 product (src/int8.rs:315-331).  K % 16 == 0, N % 4 == 0.
void launch_q8_gemm(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi, int sm_count);
// The product for a few rows with a prologue on its input rows; false: shape or row count not covered (nothing queued).
bool launch_q8_gemv_pro(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi, const GemvPro& pro);
// the most rows launch_q8_gemv_pro takes
int gemv_max_rows();

// The same product, same bits, with packed weights and packed multiply-adds (k_gemm2.cu).  false: shape not covered.
bool launch_q8_gemm2(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi, int sm_count);

// The same product for rows that are mostly zeros (spikes, k-WTA'd units): summed over the non-zero inputs only, in
// order, which gives the dense sum's bits (src/int8.rs:10-13).  false: shape not covered, use launch_q8_gemm.
// mix (may be null; EPI_ADD only, and only where event_takes_mix says so): after the add the row's dense mix of the
// streams (launch_dense_mix) is taken in the same kernel, element by element.
struct MixArgs {
    float* streams = nullptr;      // [n_streams][M * d]
    const float* w = nullptr;      // [n_streams]
    int n_streams = 0;
    // A few rows only (event_small_covers): the input row is not read from A but made in the kernel as the k winners of
    // kw_u's row (launch_kwta's arithmetic: the units at or above the k-th largest, negatives dropped, squared on
    // request), so the k winners need no kernel of their own.  kw_u == nullptr: the row comes from A as usual.
    const float* kw_u = nullptr;   // [M, K] pre-activations
    int kw_k = 0, kw_relu2 = 0;
};
bool launch_q8_event(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi, const MixArgs* mix = nullptr);
// whether launch_q8_event would take the mix along for this shape (asked first: the mix then has no kernel of its own)
bool event_takes_mix(const GemmArgs& a, GemmEpilogue epi, int n_streams);
// whether the event kernel for a few rows takes this product (only it can make the k winners itself)
bool event_small_covers(const GemmArgs& a, GemmEpilogue epi);

// The dense product on the tensor cores (tcgen05, f32 accumulate in tensor memory), for the optional fast-products
// mode: exact products (three bf16 limbs of each activation times a bf16 copy of the int8 weight), the sum in the
// tensor core's order instead of the reference's, so results agree with launch_q8_gemm to about 1e-6 of the sum of
// magnitudes and not bit for bit.
struct TcGemmArgs {
    const uint16_t* a_limbs;  // bf16 [3][M][K] from launch_split3
    const uint16_t* w_bf16;   // bf16 [N][K] from launch_widen_transpose
    const float* scale;       // [N]
    float* C;                 // [M, N], row stride ldc (a multiple of 4)
    int ldc;
    int M, N, K;
    uint32_t* status;         // ST_WAIT_TIMEOUT when a bounded wait ran out (the tile is then not written)
};
// false: shape or epilogue not covered (K % 64, N % 4, EPI_LIF) or no tensor-map encoder; nothing was launched
bool launch_tc_gemm(cudaStream_t st, const TcGemmArgs& a, GemmEpilogue epi);
void launch_split3(cudaStream_t st, const float* x, int64_t n, uint16_t* out);

// Batched f32-accurate products on the tensor cores (k_tcb.cu): C[b] = A[b] . B[b]^T with both operands as three bf16
// limbs, K-major planes [limb][batch * rows][K].
enum { TCB_STORE = 0, TCB_DECAY = 1, TCB_SCALE_ADD = 2 };
struct TcbArgs {
    const uint16_t* a;        // [3][rows_a][K], rows_a = batch * M
    const uint16_t* b;        // [3][rows_b][K], rows_b = batch * N
    int64_t rows_a, rows_b;
    int64_t a_row0, b_row0;   // first row of batch item 0 inside a plane (a window of a longer buffer)
    float* C;                 // [batch][M][ldc]
    int ldc;
    int64_t c_batch_stride;   // floats between batch items of C
    int M, N, K, batch;       // M a multiple of 128, K of 64, N of 4
    // TCB_DECAY: C = colscale[b][n] * C + A . B^T, and the new C's limbs into c_limbs [3][batch * M][N]
    const float* colscale;
    int64_t colscale_batch_stride;
    uint16_t* c_limbs;
    int64_t c_limb_plane;     // elements between limb planes
    // An optional second stretch of K from other buffers: C += A2[b] . B2[b]^T over K2 more columns (a multiple of 64), as if
    // [A | A2] and [B | B2] were single operands.  Rows of width lda2 / ldb2 elements, of which the first K2 are read.
    const uint16_t* a2;       // [3][rows_a2][lda2]
    const uint16_t* b2;       // [3][rows_b2][ldb2]
    int64_t rows_a2, rows_b2, a2_row0, b2_row0;
    int K2, lda2, ldb2;
    uint32_t* status;
};
bool launch_tc_bgemm(cudaStream_t st, const TcbArgs& a, int epi);

// The fast-weight memory over chunks of 64 tokens in its chunk-parallel form (k_chunk.cu), per-channel gates without
// momentum.  Inputs are time-major: element (token t, head-row hb, channel c) at [t * tok_stride + hb * hs + c], t in
// [0, 64 nC); HB = rows * heads.  F is the state in the step kernels' slice-major layout.
struct ChunkArgs {
    int HB, hs, nC, cw;
    int64_t tok_stride;
    const float *qn, *e, *w, *ah, *v, *la;  // unit query, unit erase direction, write key, erase key, value, log rate
    float* y;                                // reads, time-major like the inputs
    float* F;
    uint32_t* flags;                         // bit 0: a chunk's rates are outside this form's range
    uint32_t* status;
    // workspace (mem_chunk_carve)
    uint16_t *QE, *WA, *A3, *A5, *B5, *Ft_limbs;
    float *ES, *CUM, *gc, *Gm, *Qa, *Tinv, *RY, *Ft;
    uint16_t* XL;   // [3][nC * HB * 128][64]: per chunk the limbs of [T Ke; Qw], the second stretch of the state read's left operand
};
size_t mem_chunk_workspace_bytes(int HB, int hs, int nC);
void mem_chunk_carve(ChunkArgs& a, void* ws);
bool mem_chunk_covers(int hs, int T, float momentum);
bool launch_mem_chunk_scale(cudaStream_t st, const ChunkArgs& a);
bool launch_mem_chunk_rest(cudaStream_t st, const ChunkArgs& a);
int mem_chunk_launches(int nC);
void launch_widen_transpose(cudaStream_t st, const int8_t* q, int K, int N, uint16_t* out);

// ---- row kernels ----------------------------------------------------------------------------------------------
void launch_embed(cudaStream_t st, const float* tok_emb, const uint32_t* tok, int M, int d, int vocab, float* x, float* stream0, uint32_t* status,
                  const float* letters = nullptr);
// limbs (may be null): also the three bf16 limbs of y, planes [3][M * n], for launch_tc_gemm
void launch_rmsnorm(cudaStream_t st, const float* x, const float* gain, int M, int n, float* y, uint16_t* limbs = nullptr);
void launch_lif(cudaStream_t st, const float* cur, const LifParams& p, int M, int d);
// T tokens of M rows in time order: cur, spikes [T][M][d]; the state in p moves T steps
// --stp (src/model/fstep/arch_f3.rs:72-106): T tokens of M rows in time order, spikes and out [T][M][d] (out may be
// the spikes' own buffer), the synapse's state (u, x) [M][d] moves T steps
void launch_stp(cudaStream_t st, const float* spikes, const float* U, const float* F, const float* D, const float* mix, float* u, float* x, int M, int d,
                int T, float* out);
void launch_fill(cudaStream_t st, float* p, int64_t n, float v);
void launch_lif_scan(cudaStream_t st, const float* cur, const LifParams& p, int M, int d, int T, float* spikes, const float* cur_gain = nullptr);

// --dopamine / --mood (src/model/fstep/arch_f3.rs:106-186, arch_f4.rs:131-143), token-rows time-major [T][rows]:
// the surprise of every token-row from the head's logits of the position before it: s = (lse - logit[token]) * valid
// (valid: the carried flag for a chunk's first token, 1 after it), z = s * (1 / ln V) + 0.  false: vocabulary too large
// for the kernel's shared memory.
bool launch_surprise(cudaStream_t st, const float* logits, int V, const uint32_t* tok, const float* valid, int rows, int T, float* s, float* z);
// the mood's scan over a chunk's tokens from the carried mood [rows][k] (updated in place); all [T][rows][k] moods out
void launch_mood(cudaStream_t st, const float* z, int rows, int T, int k, const float* lam, const float* win, const float* bin, float* mood_state,
                 float* mood_all);
// gain [M][d] = 1 + tanh(mood [M][k] . G [k][d]) (the product in the one-row order), the LIF current's factor
void launch_mood_gain(cudaStream_t st, const float* mood_all, int k, const float* G, int M, int d, float* gain);
// --cerebellum-head (src/model/fstep/arch_f3.rs:207-283): the tokens' embedding rows gathered; the G units' sums of their
// four wired inputs of [xf, en] (en: the normed embedding rows); after the k-WTA kernel has kept the top G/32 of h into a:
// the code's list per token-row (scratch list_j, list_c [R][G], count [R]) and xf += the read-out's rows in unit order
void launch_cb_inputs(cudaStream_t st, const float* tok_emb, const uint32_t* tok, int R, int d, int V, float* emb_rows);
void launch_cb_units(cudaStream_t st, const float* xf, const float* en, const uint32_t* idx, const float* sgn, int g, int d, int R, float* h);
void launch_cb_read(cudaStream_t st, const float* a, int g, int* list_j, float* list_c, int* count, const float* W, int R, int d, float* xf);
// x += (y * (1 + tanh(z[row] w + c))) [* row_gain[row * NM_STRIDE]]: the MLP's output under --dopamine (then --neuromod's DA)
void launch_da_add(cudaStream_t st, float* x, const float* y, const float* z, const float* w, const float* c, const float* row_gain, int M, int d);

struct MemPrepArgs {
    const float* h;      // [M, d] normed input
    const float* proj;   // [M, ldp]: q | k | v | e | (g)
    int ldp;
    const float* gate_w; // [d][gate_cols]: wa1 | wb1 | wa | wb side by side, columns padded with zeros to a multiple of 4
    int gate_cols;       // padded column count (at most 256: one chain per thread)
    int gate_chunk;      // rows staged per copy; divides d, a multiple of 8
    float* be_out;       // the write strength b [M, d] as the update uses it (the token trace's side-band), or nullptr
    const float* rh_w;   // --rhythm: the write strength times rh_w[row * heads + head] before ACh; or nullptr
    const float* ach;    // --neuromod ACh: the write strength times ach[row * ach_stride], kept in [0, 2]; or nullptr
    int ach_stride;
    float* z;            // [M][gate_cols] work: h . gate_w (stage one)
    float *lra, *lrb;    // [M, d] work: the low-rank parts of the two gates (stage two)
    const float *ba, *bb, *wa2, *wb2, *off;
    const float* vres;   // [2] or nullptr
    float* v_first;      // [M, d]: written when first, read when vres
    int first;           // 1: this block's values become v_first
    int M, d, hs, rank;
    // outputs [M, d] each, qw/qa [M, d / hs]
    float *e, *v, *w, *ah, *qg, *ex, *qw, *qa;
    float* qs;           // [M, d] q * M when the memory has momentum, else nullptr
    float *qn_out, *la_out;  // [M, d] the unit query and the log rate, for the chunk-parallel form; or nullptr
    int fast;            // 1 (the tolerance mode): norms and dot products summed by a warp each, the library's exp and log
    float mom;
    uint32_t* status;
    const float* h_gain = nullptr;  // not null (a few rows only, gate_z_few_covers): h is the block's input as it came and stage one takes
                                    // its RMS norm with this gain itself, so the norm needs no kernel of its own
};
// out [M][n] = x [M][d] . W [d][n] in gemm's one-row order (an fma chain down the rows from the first product), the weights
// staged through shared memory for a few rows at a time; n a multiple of 4 (at most 224), d a multiple of chunk
void launch_chain_gemv(cudaStream_t st, const float* x, const float* W, int M, int d, int n, int chunk, float* out, const float* norm_gain = nullptr);
// whether the kernel for a few rows takes this projection (only it can take the input's norm itself)
bool gate_z_few_covers(const float* x, const float* W, int M, int d, int n);
// whether launch_q8_gemv_pro would take this product (asked before anything is queued)
bool q8_gemv_pro_covers(const GemmArgs& a, const GemvPro& pro);
// --dendrite (src/model/fstep/arch_f4.rs:120-141): act [M][H] *= 1 + tanh(z1 [M][rank] . B [rank][H]), the product in gemm's
// one-row order
void launch_dend_gain(cudaStream_t st, const float* z1, int rank, const float* B, int M, int H, float* act);
// --neuromod: sig [M][4] = 2 sigmoid(z [M][4] + bias [k]) for the first k of each row's four
void launch_nucleus(cudaStream_t st, const float* z, const float* bias, int k, int M, float* sig);
// x += y, elementwise
void launch_add_into(cudaStream_t st, float* x, const float* y, int64_t n, const float* row_gain = nullptr, int d = 0);
// --thalamus: the relay takes one 16-wide read per token-row into its sum and gives the next block's gates [M][NM_STRIDE]
// ([0] residual, [1] memory read); then the residual rule on a block's whole change (src/model/fstep/arch_f2.rs:62-153)
void launch_relay(cudaStream_t st, const float* thr, float* acc, bool first, int reads, const float* G, const float* bias, int M, float* g);
void launch_relay_res(cudaStream_t st, float* x, const float* x_in, const float* g, int M, int d);
// three launches: the gates' first projection, their low-rank second stage, then everything per row
void launch_mem_prep(cudaStream_t st, const MemPrepArgs& a);
// the same in its two parts: the gates' projection stages (need only a.h), then the per-row kernel (needs a.proj too)
void launch_mem_gates(cudaStream_t st, const MemPrepArgs& a);
void launch_mem_gates_low(cudaStream_t st, const MemPrepArgs& a);  // stage two alone, when a.z was made elsewhere
void launch_mem_prep_rows(cudaStream_t st, const MemPrepArgs& a);

struct MemHeadsArgs {
    float* f;            // this block's fast weights, slice-major: [M][nh][hs / cw][hs][cw] f32, updated in place
    float* s;            // the momentum matrix, same layout, or nullptr (multi-token kernel only)
    const float* qs;     // [M, nh * hs] q * M (momentum only)
    float mom;           // M
    int M, nh, hs, cw, chunk_rows;
    const float *e, *v, *w, *ah, *qg, *ex;  // [M, nh * hs]
    const float *qw, *qa;                    // [M, nh]
    float* y;                                // [M, nh * hs]
    uint32_t* status;
    uint32_t wait_limit;                     // polls before a bounded wait gives up (0: the kernel's default)
    int fault_chunk_plus1;                   // testing aid: c + 1 makes every block expect 16 bytes too many for chunk c of its
                                             // first item, so that barrier never completes and the wait runs out (0: off)
};
// T tokens in time order with a block's slice of the state resident in shared memory between them: the vectors and y
// are time-major [T][M][nh * hs], qw/qa [T][M][nh]; the state is read and written once for the whole chunk.
void launch_mem_heads_seq(cudaStream_t st, const MemHeadsArgs& a, int T);

// One token as a single streaming pass (k_stream.cu): the token's read, while the update the token BEFORE it left
// pending is applied to the rows as they stream by; this token's own update stays pending (its alpha, w, ah per row
// and value, rr per column).  The state in HBM is therefore one update behind until launch_mem_flush applies the
// pending update alone.  Same bits as the resident form.
struct MemStreamArgs {
    float* f;                       // this block's fast weights, slice-major [M][nh][hs / cw][hs][cw]
    float* f_out;                   // where the updated weights are written (nullptr: in place); used only with a pending update
    int M, nh, hs, cw;
    int parts;                      // set by the launcher: blocks a head's columns are split over
    const float *e, *qg, *v;        // this token: [M, nh * hs]
    const float *qw, *qa;           // this token: [M, nh]
    float* y;                       // [M, nh * hs]
    float* rr_out;                  // [M, nh * hs]: this token's rr (part of its pending update)
    const float *px, *pw, *pah;     // the pending update's alpha, w, ah per row [M, nh * hs]; px == nullptr: none pending
    const float *pv, *prr;          // the pending update's value and rr per column [M, nh * hs]
    int early_state;                // 1: nothing queued just before this pass writes the state (a decode step), so the few-row kernel may request it before
                                    // its wait for the kernel before
};
bool launch_mem_stream(cudaStream_t st, const MemStreamArgs& a);
void launch_mem_flush(cudaStream_t st, float* f, const float* px, const float* pw, const float* pah, const float* pv, const float* prr, int64_t heads,
                      int hs, int cw);
// the column-slice width and the rows per bulk copy the kernel uses for a head size; false: head size not covered
bool mem_heads_tiling(int hs, int* cw, int* chunk_rows, bool momentum = false);
// natural [heads][hs][hs] to slice-major [heads][hs / cw][hs][cw] (to_slices 1) or back (0)
void launch_retile(cudaStream_t st, const float* src, float* dst, int64_t heads, int hs, int cw, int to_slices);

// rh_r: --rhythm's gain of the read [M][heads], after the head norm and before the output gate; or nullptr
void launch_mem_post(cudaStream_t st, const float* y_raw, const float* gate, int ldg, int M, int d, int hs, float* y, uint16_t* limbs = nullptr,
                     const float* rh_r = nullptr);
// --rhythm (src/model/fstep/arch_f4.rs:47-107), token-rows time-major [T][rows]: from the reset read-outs pre [M][4] (two
// used, bias not yet added) the clocks' times token after token from the carried ones [rows][2] (updated in place) and
// the phase features f [M][4] = cos, sin of time * exp(lw); then a block's gains per head 1 + tanh(f G) [M][heads] twice
void launch_rhythm(cudaStream_t st, const float* pre, const float* br, const float* lw, int rows, int T, float* times, float* f);
void launch_rhythm_gates(cudaStream_t st, const float* f, const float* Gw, const float* Gr, int M, int nh, float* gw, float* gr);

struct EngramArgs {
    const float* qkv;    // [M, 3 d]
    void* k;             // [M, heads, cap, hs] bf16 or f32
    void* v;
    int32_t* n;          // [M] tokens held
    int32_t* start;      // [M] ring start
    int M, d, hs, cap, keep, bf16;   // cap: ring slots per head; keep: tokens kept after the read (oldest dropped)
    float* o;            // [M, d]
    uint32_t* status;
};
// returns false when n_max keys do not fit the kernel's shared memory
bool launch_engram(cudaStream_t st, const EngramArgs& a, int n_max);

// The long-store form: append, then per (row, head, segment of seg_len keys) partial softmax statistics
// [row][head][n_seg][2 + hs] = (max, sum, unnormalised mix), merged in position order by the combine kernel (which
// also merges the parts gathered from several GPUs).  Agrees with the single-pass read to rounding, not bit for bit.
void launch_engram_append(cudaStream_t st, const EngramArgs& a);
void launch_engram_trim(cudaStream_t st, const EngramArgs& a);
int engram_segments(int n_max, int seg_len);
bool engram_fits_one_block(int d, int hs, int n_max);
bool launch_engram_partial(cudaStream_t st, const EngramArgs& a, int seg_len, int n_seg, float* partial);
void launch_engram_combine(cudaStream_t st, const float* partial, int M, int nh, int hs, int n_part, float* o, int n_groups = 1);

// The engram over a whole prompt chunk on the tensor cores (k_eattn.cu): the chunk's T keys and values join the store,
// every token's causal read, the counts move on by T.  qkv [T][M][3 d] and o [T][M][d] are time-major; the store must
// not wrap or trim inside the chunk (start + n + T <= cap for every row: the caller checks on its mirror of the counts).
struct EngramChunkArgs {
    const float* qkv;
    float* o;
    void* k;             // [M, heads, cap, hs] bf16
    void* v;
    int32_t* n;
    int32_t* start;
    int M, d, hs, cap, T, bf16;
    uint32_t* status;
};
bool launch_engram_chunk(cudaStream_t st, const EngramChunkArgs& a);

// limbs (may be null): also the three bf16 limbs of the output, planes [3][M * n], for launch_tc_gemm
void launch_kwta(cudaStream_t st, const float* u, int M, int n, int k, int relu2, float* a, uint16_t* limbs = nullptr);
// x <- x + sum_j streams[j] * w[j] over the n_streams streams (the last one is x itself, stored first)
void launch_dense_mix(cudaStream_t st, float* x, float* streams, const float* w, int n_streams, int64_t MD);
// `diary::pick` for every row: softmax(logits / temperature), the top_k most likely, one draw with the row's uniform
// number in [0, 1).  false: not covered (top_k above 1024, a vocabulary too large for shared memory, temperature <= 0).
bool launch_sample(cudaStream_t st, const float* logits, int M, int V, float temperature, int top_k, const double* uniform, uint32_t* next);
// whether launch_sample covers a vocabulary and a top_k (asked before a step moves the state, and once per generation)
bool sample_covered(int V, int top_k);
// the largest vocabulary launch_surprise holds in shared memory
constexpr int SURPRISE_MAX_VOCAB = 220 * 1024 / 4;
void launch_argmax(cudaStream_t st, const float* logits, int M, int V, uint32_t* next);
void launch_math(cudaStream_t st, int which, const float* x, int64_t n, float* y);
void launch_round_bf16(cudaStream_t st, const float* x, int64_t n, uint16_t* y);
void launch_widen_bf16(cudaStream_t st, const uint16_t* x, int64_t n, float* y);

}  // namespace ava
