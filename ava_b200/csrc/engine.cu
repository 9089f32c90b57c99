// Host side of the B200 engine for Ava's per-token block step: the model's weights and the carried state in device
// memory, the launch sequence of one step, and the C ABI of include/ava_engine.h.
//
// The step follows the reference's fused one-token step (design-tests/nn/gpu/src/model/fstep/arch.rs:525-1073) for
// every row of a state at once; the rows are independent (src/state.rs:13-15).  Unlike the reference, which computes
// everything and commits at the end (arch.rs:1059-1069), the state is updated in place as the step goes: a step that
// reports a non-finite gate or key (AVA_ERR_NONFINITE) has already moved the state.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "../../include/ava_engine.h"
#include "ava_math.h"
#include "kernels.cuh"
#include "nccl_dl.h"

namespace {

using namespace ava;

thread_local std::string g_create_error;

// ------------------------------------------------------------------------------------------------ device memory
struct Dev {
    void* p = nullptr;
    size_t bytes = 0;
    Dev() = default;
    Dev(const Dev&) = delete;
    Dev& operator=(const Dev&) = delete;
    ~Dev() { release(); }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        bytes = 0;
    }
    cudaError_t alloc(size_t n) {
        release();
        if (n == 0) return cudaSuccess;
        const cudaError_t e = cudaMalloc(&p, n);
        if (e == cudaSuccess) bytes = n;
        return e;
    }
    template <typename T>
    T* as() const { return reinterpret_cast<T*>(p); }
};

struct QMat {
    int din = 0, dout = 0;
    Dev q, scale;
    Dev wt;  // fast-products mode only: the weights as bf16 [dout][din]
    const int8_t* qp() const { return q.as<int8_t>(); }
    const float* sp() const { return scale.as<float>(); }
};

struct HostQ {
    int din = 0, dout = 0;
    std::vector<int8_t> q;
    std::vector<float> scale;
};

struct BlockDev {
    Dev mem_norm, beta, theta, rho, again, hebb_norm, gate_w, ba, bb, wa2, wb2, off, vres, eng_norm, mlp_norm, dense;
    Dev stp_U, stp_F, stp_D, stp_mix;  // --stp: sigmoids of the synapse's parameters, and its mix
    Dev dend_a, dend_b;                // --dendrite: A [d][32], B [32][hidden]
    Dev rh_w, rh_r;                    // --rhythm: the write strength's and the read's gates [4][heads]
    Dev da_w, da_c, mood_g;            // --dopamine: gate [d] twice; --mood: gain [k][d] (blocks after the first)
    Dev gate_wl;                       // fast products: the three bf16 limbs of gate_w transposed, [3][gate_cols][d]
    QMat win, wout, proj, wo, eqkv, ewo, w1, w2;
};

// nn/parts/src/quant.rs:18-31
void quantize_int8(const float* w, int rows, int cols, int8_t* q, float* scale) {
    for (int c = 0; c < cols; ++c) scale[c] = 0.f;
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) scale[c] = std::max(scale[c], std::fabs(w[(size_t)r * cols + c]));
    for (int c = 0; c < cols; ++c) scale[c] = scale[c] > 0.f ? scale[c] / 127.0f : 1.0f;
    for (size_t i = 0; i < (size_t)rows * cols; ++i) {
        float v = std::round(w[i] / scale[i % cols]);
        q[i] = (int8_t)std::min(std::max(v, -127.0f), 127.0f);
    }
}

}  // namespace

// ================================================================================================ engine
// The work buffers of one lane of rows.  The engine itself is lane 0; a decode step of a large batch may run its rows
// as several lanes, each a contiguous window of the state's rows with buffers and a stream of its own, so that one
// lane's latency-bound kernels run beside another lane's.
struct Work {
    int ws_rows = 0;
    Dev x, h, proj, ve, vv, vw, vah, vqg, vex, vqs, qw, qa, yraw, y, eqkv, eo, u, act, streams, v_first;
    Dev gz, lra, lrb;  // the gates' stages: [rows][gate_cols], [rows][d] twice
    Dev vqn, vla, chunk_ws, chunk_flag;  // the chunk-parallel memory of the tolerance mode: unit queries, log rates, its work space
    Dev vrr;                             // a chunk of tokens through the streaming pass: every token's rr [T][rows][d]
    Dev limbs;                           // fast products: [3][rows][K] bf16 limbs of the current product's input
    const float* limbs_src = nullptr;    // the f32 buffer whose limbs the producing kernel has just written there
    int limbs_rows = 0;
    Dev sig;           // --neuromod: [rows][4] NE, ACh, DA (and one unused) of the step's token-rows
    // --dopamine / --mood: block 0's normed output [rows][d], the rows the head reads (the position before each), the
    // head's logits for them [rows][vocab], surprise s and z [rows], moods [rows][k], the current's gain and the MLP's output [rows][d]
    Dev sur_xf, sur_in, sur_logits, sur_s, sur_z, mood_all, mood_gain, y2;
    Dev cb_emb, cb_en, cb_h, cb_a, cb_lj, cb_lc, cb_n;  // --cerebellum-head: embedding rows (raw, normed) [rows][d], units and kept units
                                                        // [rows][G], the code's list [rows][G] twice, its length [rows]
    Dev side;                // [rows][d] scratch of the token trace's side-band (only while intermediates are kept)
    Dev rh_f, rh_gw, rh_gr;  // --rhythm: phase features [rows][4], the block's gains per head [rows][heads] twice
    Dev th_acc, th_g, x_in;  // --thalamus: the relay's sum [rows][16], the block's gates [rows][4], the block's input [rows][d]
    Dev ctx, dz1;        // --dendrite: the block's memory read [rows][d], its projection [rows][32]
    Dev eng_partial;         // [rows][heads][segments][2 + hs] partial softmax statistics of the segmented read
    cudaStream_t lane_stream = nullptr;  // lanes after the first: the stream their kernels are queued on
    cudaEvent_t lane_done = nullptr;
    cudaStream_t side_stream = nullptr;  // the lane's side stream: the gates' projections run there beside the q|k|v|e|g product
    cudaEvent_t side_go = nullptr, side_done = nullptr;
};

struct ava_engine : Work {
    ava_config cfg{};
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    bool finalized = false;
    mutable std::string err;
    std::string blocker;
    int64_t launches = 0;
    uint64_t fingerprint = 0;

    std::map<std::string, std::vector<float>> host_f32;
    std::map<std::string, HostQ> host_q8;

    Dev tok_emb, final_norm;
    Dev nm_norm, nm_wn, nm_bn;  // --neuromod: the nucleus (gain [d], read-out padded to [d][4], bias [k])
    Dev rhy_lw, rhy_wr, rhy_br;        // --rhythm: log frequencies [2], reset read-out padded to [d][4], bias [2]
    Dev mood_lam, mood_win, mood_bin;  // --mood: decay, input weight and bias [k]
    Dev letters;                    // --letters: every token's share of its input [vocab][d], built when the engine is finalized
    std::vector<uint8_t> tok_bytes;  // the tokens' spellings, bytes[tok_off[t] .. tok_off[t + 1])
    std::vector<int64_t> tok_off;
    Dev cb_w, cb_idx, cb_sgn;       // --cerebellum-head: read-out [G][d], wiring [G][4] (u32 inputs, f32 weights)
    Dev th_read, th_gate, th_bias;  // --thalamus: reads [blocks][d][16], gates [blocks][16][2], biases [blocks][2]
    QMat head;
    std::vector<std::unique_ptr<BlockDev>> blocks;
    int cw = 0, rb = 0;  // fast-weight slice width and rows per bulk copy
    int gate_cols = 0, gate_chunk = 0;  // the gates' projection matrix: padded columns, rows per staged chunk

    // the engine's own (lane 0's) work buffers are the members of Work; these belong to the engine as a whole
    int ws_logit_rows = 0;
    Dev logits, tok, next, status;
    Dev uniform;       // [rows] f64: the sampler's draws of one step
    Dev ones;          // a vector of ones [d] (the gain of a plain RMS norm)
    std::vector<std::unique_ptr<Work>> more_lanes;  // lanes 1, 2, ... (lane 0 is the engine itself)
    bool gemm2 = true;                              // dense products of more than a few rows through the packed-weight kernel (k_gemm2.cu)
    int n_lanes = 2;                                // lanes a decode step of enough rows is split into (ava_engine_set_lanes)
    cudaEvent_t fork_ev = nullptr;
    cudaStream_t cur = nullptr;                     // the stream the launch helpers queue on (the lane being queued)
    uint32_t* status_host = nullptr;  // pinned

    bool prof = false;
    bool prof_lanes = std::getenv("AVA_TIMELINE") != nullptr;  // tuning aid: keep the lanes under the section clock (its per-kernel sums then overlap)
    struct Pending { const char* cls; cudaEvent_t a, b; cudaStream_t st; };
    std::vector<Pending> prof_pending;
    std::map<std::string, std::pair<int64_t, double>> prof_total;  // kernel -> (launches, milliseconds)

    bool fast = false;     // dense products on the tensor cores (exact products, the tensor core's summation order)
    bool chunk_mem = true; // with fast: a prompt chunk's fast-weight memory in the chunk-parallel form (k_chunk.cu)
    int64_t chunked_blocks = 0, chunk_fallbacks = 0, chunked_reads = 0;
    Work* cur_w = nullptr; // the lane being queued (its work buffers; set with `cur`)

    int long_seg = 0;      // > 0: the engram is always read in segments of this many keys (else only when it must be)

    bool keep = false;
    std::map<std::pair<std::string, int>, std::unique_ptr<Dev>> debug;
    std::map<std::string, int64_t> debug_width;
    int debug_rows = 0;

    int nh() const { return cfg.d / cfg.head_size; }
    int proj_w() const { return (cfg.out_gate ? 5 : 4) * cfg.d; }

    int fail(int code, const char* fmt, ...) const {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        err = buf;
        return code;
    }
    int cuda_fail(cudaError_t e, const char* what) const { return fail(AVA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e)); }
};

struct ava_state {
    ava_engine* e = nullptr;
    int rows = 0;
    int ring = 0;   // engram slots per head
    int keep = 0;   // tokens kept after a read
    Dev lif_v, lif_s, lif_a;  // [L][rows][d]
    Dev mem_f;                // [L][rows][nh][hs / cw][hs][cw]: slice-major, a block of threads owns one contiguous slice
    Dev mem_s;                // the momentum matrix, same layout (only with --mem-momentum)
    // The plain memory's decode pass (k_stream.cu) leaves each token's update pending: alpha, w, ah per row and value,
    // rr per column of every block, [2][5][L][rows][d] (two sets that take turns: one is written by this step while the
    // other, the step before's, is applied).  mem_f is one update behind while `pending` is set; flush_pending()
    // brings it up to date for every other reader.
    Dev pend;
    // Commit at the end (ava_state_set_commit_at_end): a second copy of the fast weights that a one-token step writes while
    // it reads the first (the two change places when the call has succeeded), and room for a copy of the small carried
    // tensors taken before a call.
    bool commit_at_end = false, txn_pingpong = false;
    Dev mem_f_alt, snap;
    bool pending = false;
    int pend_set = 0;         // the set the LAST step wrote
    float* pend_at(int set, int what, int block) { return pend.as<float>() + ((((size_t)set * 5 + what) * e->cfg.n_blocks + block) * rows) * e->cfg.d; }
    Dev stp_u, stp_x;         // [L][rows][d]: the synapse's (u, x) (only with --stp; a fresh state has u = 0, x = 1)
    Dev rh;                                   // --rhythm: the time since each clock's last reset [rows][2]
    Dev sur_prev, sur_valid, sur_last, mood;  // --dopamine / --mood: block 0's last normed output [rows][d], whether there is one
                                              // [rows], the last surprise [rows], the mood [rows][k] (all zero in a fresh state)
    Dev eng_k, eng_v;         // [rows][enh][ring][ehs]
    Dev eng_n, eng_start;     // [rows] i32
    std::vector<int32_t> n_host, start_host;
    std::vector<int64_t> seen;
    // a store split by position over several GPUs: this state keeps the tokens rank `shard_rank` owns
    int shard_world = 0, shard_rank = 0;
    int64_t shard_block = 0, shard_pos = 0;
    size_t kv_elem() const { return e->cfg.eng_store_bf16 ? 2 : 4; }
};

namespace {

#define CK(call)                                                   \
    do {                                                           \
        const cudaError_t e__ = (call);                            \
        if (e__ != cudaSuccess) return e->cuda_fail(e__, #call);   \
    } while (0)

bool split_block_name(const std::string& name, int n_blocks, int* block, std::string* rest) {
    if (name.size() < 3 || name[0] != 'b') return false;
    const size_t dot = name.find('.');
    if (dot == std::string::npos || dot < 2) return false;
    for (size_t i = 1; i < dot; ++i)
        if (name[i] < '0' || name[i] > '9') return false;
    *block = std::atoi(name.substr(1, dot - 1).c_str());
    *rest = name.substr(dot + 1);
    return *block >= 0 && *block < n_blocks;
}

// expected float count of an f32 tensor, or -1 for an unknown name
int64_t f32_len(const ava_config& c, const std::string& name) {
    const int64_t d = c.d, nh = c.d / c.head_size, r = c.gate_rank;
    if (name == "tok_emb") return (int64_t)c.vocab * d;
    if (name == "final.norm") return d;
    if (name == "nm.norm" && c.neuromod > 0) return d;
    if (name == "nm.wn" && c.neuromod > 0) return d * c.neuromod;
    if (name == "nm.bn" && c.neuromod > 0) return c.neuromod;
    if (c.rhythm && (name == "v51.rhythm.lw" || name == "v51.rhythm.br")) return 2;
    if (c.rhythm && name == "v51.rhythm.wr") return d * 2;
    if (c.mood > 0 && (name == "v51.mood.lam" || name == "v51.mood.win" || name == "v51.mood.bin")) return c.mood;
    if (c.letters) {  // LETTER_DIM 64, LETTER_MAX 16 (src/v51.rs:54-55)
        if (name == "v51.letters.byte") return 256 * 64;
        if (name == "v51.letters.pos" || name == "v51.letters.end") return 16 * 64;
        if (name == "v51.letters.wo") return 64 * d;
    }
    if (name == "cbh.wo" && c.cb_units > 0) return (int64_t)c.cb_units * d;
    if (name == "th.read" && c.thalamus) return (int64_t)c.n_blocks * d * 16;  // TH_K (src/v51b.rs:45)
    if (name == "th.gate" && c.thalamus) return (int64_t)c.n_blocks * 16 * 2;
    if (name == "th.bias" && c.thalamus) return (int64_t)c.n_blocks * 2;
    int b;
    std::string rest;
    if (!split_block_name(name, c.n_blocks, &b, &rest)) return -1;
    static const char* vec_d[] = {"mem.norm", "mem.beta", "mem.theta", "mem.arho", "mem.again", "hebb.norm", "hebb.off", "eng.norm", "mlp.norm",
                                  "parts.stp.u_param", "parts.stp.f_param", "parts.stp.d_param", "parts.stp.mix"};
    for (const char* n : vec_d)
        if (rest == n) return d;
    if ((rest == "v51.da_w" || rest == "v51.da_c") && c.dopamine && b > 0) return d;
    if (rest == "v51.mood_g" && c.mood > 0 && b > 0) return (int64_t)c.mood * d;
    if ((rest == "v51.rh_w" || rest == "v51.rh_r") && c.rhythm && c.fast_mem) return 4 * nh;
    if (rest == "v51.dend_a") return d * 32;  // DEND_RANK (src/v51.rs:52)
    if (rest == "v51.dend_b") return (int64_t)32 * c.hidden;
    if (rest == "hebb.wa" || rest == "hebb.wb") return d * nh;
    if (rest == "hebb.ba" || rest == "hebb.bb") return nh;
    if (rest == "hebb.wa1" || rest == "hebb.wb1" || rest == "hebb.wa2" || rest == "hebb.wb2") return d * r;
    if (rest == "hebb.vres") return 2;
    if (rest == "dense") return b + 2;
    return -1;
}

bool q8_dims(const ava_config& c, const std::string& name, int* din, int* dout) {
    if (name == "head") {
        *din = c.d;
        *dout = c.vocab;
        return true;
    }
    int b;
    std::string rest;
    if (!split_block_name(name, c.n_blocks, &b, &rest)) return false;
    static const char* sq[] = {"mem.win", "mem.wout", "hebb.wq", "hebb.wk", "hebb.wv", "hebb.we", "hebb.wg", "hebb.wo", "eng.wq", "eng.wk", "eng.wv", "eng.wo"};
    for (const char* n : sq)
        if (rest == n) {
            *din = *dout = c.d;
            return true;
        }
    if (rest == "mlp.w1") {
        *din = c.d;
        *dout = c.hidden;
        return true;
    }
    if (rest == "mlp.w2") {
        *din = c.hidden;
        *dout = c.d;
        return true;
    }
    return false;
}

int upload(ava_engine* e, Dev& dst, const void* src, size_t bytes) {
    CK(dst.alloc(bytes));
    CK(cudaMemcpy(dst.p, src, bytes, cudaMemcpyHostToDevice));
    return AVA_OK;
}

int upload_f32(ava_engine* e, Dev& dst, const std::string& name, bool need) {
    auto it = e->host_f32.find(name);
    if (it == e->host_f32.end()) return need ? e->fail(AVA_ERR_MISSING, "missing tensor %s", name.c_str()) : AVA_OK;
    return upload(e, dst, it->second.data(), it->second.size() * sizeof(float));
}

// the int8 copies of `names` side by side [din, sum of douts] (src/int8.rs:86-102)
int upload_q8(ava_engine* e, QMat& dst, const std::vector<std::string>& names) {
    int din = 0, dout = 0;
    for (const std::string& n : names) {
        auto it = e->host_q8.find(n);
        if (it == e->host_q8.end()) return e->fail(AVA_ERR_MISSING, "missing int8 matrix %s", n.c_str());
        if (din && it->second.din != din) return e->fail(AVA_ERR_ARG, "%s: input width differs from its neighbours", n.c_str());
        din = it->second.din;
        dout += it->second.dout;
    }
    std::vector<int8_t> q((size_t)din * dout);
    std::vector<float> sc(dout);
    int c0 = 0;
    for (const std::string& n : names) {
        const HostQ& hq = e->host_q8[n];
        for (int j = 0; j < din; ++j) std::memcpy(&q[(size_t)j * dout + c0], &hq.q[(size_t)j * hq.dout], hq.dout);
        std::copy(hq.scale.begin(), hq.scale.end(), sc.begin() + c0);
        c0 += hq.dout;
    }
    dst.din = din;
    dst.dout = dout;
    int rc = upload(e, dst.q, q.data(), q.size());
    if (rc) return rc;
    return upload(e, dst.scale, sc.data(), sc.size() * sizeof(float));
}

const char* find_blocker(const ava_config& c, int* cw, int* rb) {
    if (c.d <= 0 || c.n_blocks <= 0 || c.vocab <= 0 || c.hidden <= 0 || c.head_size <= 0 || c.d % c.head_size) return "bad shape";
    if (c.d % 16 || c.hidden % 16) return "widths must be multiples of 16 (the product kernel's k step)";
    if (c.vocab % 4) return "vocabulary must be a multiple of 4";
    if (c.gate_rank < 1) return "gate rank must be at least 1";
    if (c.eng_block >= 0 && (c.eng_head_size <= 0 || c.d % c.eng_head_size)) return "bad engram head size";
    if (c.spikes < 0 || c.spikes > 2) return "unknown spike kind";
    if (c.neuromod != 0 && (c.neuromod < 2 || c.neuromod > 4)) return "neuromod: 2 to 4 signals";
    if (c.mood < 0 || c.mood > 16) return "mood: up to 16 units";
    if (c.cb_units < 0 || c.cb_units % 32) return "cerebellum head: a multiple of 32 units";
    if (c.rhythm && !c.fast_mem) return "rhythm: a part of the blocks with the fast-weight memory";
    if (c.thalamus && !c.fast_mem) return "thalamus: a part of the blocks with the fast-weight memory";
    if ((c.dopamine || c.mood > 0) && c.vocab > SURPRISE_MAX_VOCAB) return "dopamine / mood: the surprise kernel holds a vocabulary of up to 56320 in shared memory";
    if (c.fast_mem && (c.head_size % 16 || !mem_heads_tiling(c.head_size, cw, rb, c.mem_momentum > 0.0f))) return "memory head size not covered (a multiple of 16 whose column slice fits shared memory)";
    return nullptr;
}

int ensure_workspace(ava_engine* e, Work& w, int rows, int logit_rows = 0) {
    if (logit_rows > e->ws_logit_rows) {
        CK(e->logits.alloc((size_t)logit_rows * e->cfg.vocab * sizeof(float)));
        e->ws_logit_rows = logit_rows;
    }
    if (rows <= w.ws_rows) return AVA_OK;
    const ava_config& c = e->cfg;
    const size_t M = rows, d = c.d, f = sizeof(float);
    CK(w.x.alloc(M * d * f));
    CK(w.h.alloc(M * d * f));
    CK(w.proj.alloc(M * e->proj_w() * f));
    for (Dev* b : {&w.ve, &w.vv, &w.vw, &w.vah, &w.vqg, &w.vex, &w.yraw, &w.y, &w.eo, &w.v_first}) CK(b->alloc(M * d * f));
    if (c.mem_momentum > 0.0f) CK(w.vqs.alloc(M * d * f));
    CK(w.gz.alloc(M * std::max(e->gate_cols, 16) * f));
    CK(w.lra.alloc(M * d * f));
    CK(w.lrb.alloc(M * d * f));
    CK(w.qw.alloc(M * e->nh() * f));
    CK(w.qa.alloc(M * e->nh() * f));
    CK(w.eqkv.alloc(M * 3 * d * f));
    CK(w.u.alloc(M * c.hidden * f));
    CK(w.act.alloc(M * c.hidden * f));
    CK(w.streams.alloc(c.dense ? (size_t)(c.n_blocks + 1) * M * d * f : 0));
    if (&w == static_cast<Work*>(e)) {  // the engine's own token, next-token and draw buffers cover all lanes' rows
        CK(e->tok.alloc(M * sizeof(uint32_t)));
        CK(e->next.alloc(M * sizeof(uint32_t)));
        CK(e->uniform.alloc(M * sizeof(double)));
    }
    if (c.neuromod > 0) CK(w.sig.alloc(M * 4 * f));
    if (c.dopamine || c.mood > 0) {
        CK(w.sur_xf.alloc(M * d * f));
        CK(w.sur_in.alloc(M * d * f));
        CK(w.sur_logits.alloc(M * c.vocab * f));
        CK(w.sur_s.alloc(M * f));
        CK(w.sur_z.alloc(M * f));
        if (c.mood > 0) {
            CK(w.mood_all.alloc(M * c.mood * f));
            CK(w.mood_gain.alloc(M * d * f));
        }
        if (c.dopamine) CK(w.y2.alloc(M * d * f));
    }
    if (c.cb_units > 0) {
        const size_t G = c.cb_units;
        CK(w.cb_emb.alloc(M * d * f));
        CK(w.cb_en.alloc(M * d * f));
        CK(w.cb_h.alloc(M * G * f));
        CK(w.cb_a.alloc(M * G * f));
        CK(w.cb_lj.alloc(M * G * sizeof(int)));
        CK(w.cb_lc.alloc(M * G * f));
        CK(w.cb_n.alloc(M * sizeof(int)));
    }
    if (c.rhythm) {
        CK(w.rh_f.alloc(M * 4 * f));
        CK(w.rh_gw.alloc(M * e->nh() * f));
        CK(w.rh_gr.alloc(M * e->nh() * f));
    }
    if (c.thalamus) {
        CK(w.th_acc.alloc(M * 16 * f));
        CK(w.th_g.alloc(M * 4 * f));
        CK(w.x_in.alloc(M * d * f));
    }
    if (c.dendrite && c.fast_mem) {
        CK(w.ctx.alloc(M * d * f));
        CK(w.dz1.alloc(M * 32 * f));
    }
    w.ws_rows = rows;
    return AVA_OK;
}

// Section clock (the reference's fused step has one too: src/model/fstep/arch.rs:131-165): with profiling on, every
// kernel launch is bracketed by CUDA events on the engine's stream; ava_prof_read folds them into per-kernel totals.
void prof_begin(ava_engine* e, const char* cls) {
    if (!e->prof) return;
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
    cudaEventRecord(a, e->cur);
    e->prof_pending.push_back({cls, a, b, e->cur});
}
void prof_end(ava_engine* e) {
    e->launches++;
    if (!e->prof || e->prof_pending.empty()) return;
    cudaEventRecord(e->prof_pending.back().b, e->cur);
}

void dbg(ava_engine* e, const char* name, int block, const float* src, int rows, int64_t width) {
    if (!e->keep) return;
    auto& slot = e->debug[{name, block}];
    if (!slot) slot.reset(new Dev());
    const size_t bytes = (size_t)rows * width * sizeof(float);
    if (slot->bytes != bytes) slot->alloc(bytes);
    cudaMemcpyAsync(slot->p, src, bytes, cudaMemcpyDeviceToDevice, e->cur);
    e->debug_width[name] = width;
    e->debug_rows = rows;
}

// fast products: where the kernel that writes `dst` [M, K] should also leave its bf16 limbs (null when the mode is off)
uint16_t* limbs_for(ava_engine* e, const float* dst, int M, int K) {
    if (!e->fast || K % 64) return nullptr;
    const size_t need = (size_t)3 * M * K * sizeof(uint16_t);
    if (e->cur_w->limbs.bytes < need && e->cur_w->limbs.alloc(need) != cudaSuccess) return nullptr;
    e->cur_w->limbs_src = dst;
    e->cur_w->limbs_rows = M;
    return e->cur_w->limbs.as<uint16_t>();
}

int gemm(ava_engine* e, const char* cls, const float* A, int lda, const QMat& w, float* C, int ldc, int M, GemmEpilogue epi, const LifParams* lif = nullptr, bool sparse = false,
         const float* row_gain = nullptr, bool int_rows = false, const GemvPro* pro = nullptr, MixArgs* mix = nullptr) {
    GemmArgs g{};
    g.A = A;
    g.lda = lda;
    g.W = w.qp();
    g.ldw = w.dout;
    g.scale = w.sp();
    g.C = C;
    g.ldc = ldc;
    g.M = M;
    g.N = w.dout;
    g.K = w.din;
    if (lif) g.lif = *lif;
    if (epi == EPI_ADD) g.lif.ne = row_gain;  // [rows][NM_STRIDE]
    if (pro && pro->kind != PRO_NONE) {
        // a few rows, the input's norm taken inside the product: AVA_NOT_APPLICABLE (nothing queued) sends the caller
        // to the norm's own kernel and the plain product
        if (e->fast || sparse || M > gemv_max_rows()) return AVA_NOT_APPLICABLE;
        prof_begin(e, cls);
        const bool queued = launch_q8_gemv_pro(e->cur, g, epi, *pro);
        prof_end(e);
        if (!queued) e->launches--;
        return queued ? AVA_OK : AVA_NOT_APPLICABLE;
    }
    // Rows of small integers (spikes) times int8 weights on the tensor cores, one bf16 limb each side: every product and
    // partial sum is an integer below 2^24, so the f32 accumulator is exact in any order and the result is the event
    // sum's bits.  Taken for a prompt chunk when the bf16 copy of the weights exists (fast products on).
    if (int_rows && e->fast && w.wt.p && M >= 1024 && M % 128 == 0 && epi == EPI_ADD && !row_gain && lda == w.din && ldc == w.dout && w.din % 64 == 0 &&
        w.dout % 4 == 0) {
        const size_t need = (size_t)M * w.din * sizeof(uint16_t);
        if (e->cur_w->limbs.bytes < need) CK(e->cur_w->limbs.alloc(need));
        e->cur_w->limbs_src = nullptr;
        prof_begin(e, "tc.round");
        launch_round_bf16(e->cur, A, (int64_t)M * w.din, e->cur_w->limbs.as<uint16_t>());
        prof_end(e);
        TcbArgs t{};
        t.a = e->cur_w->limbs.as<uint16_t>(); t.rows_a = M; t.b = w.wt.as<uint16_t>(); t.rows_b = w.dout;
        t.C = C; t.ldc = ldc; t.M = M; t.N = w.dout; t.K = w.din; t.batch = 1;
        t.colscale = w.sp(); t.status = e->status.as<uint32_t>();
        prof_begin(e, cls);
        const bool launched = launch_tc_bgemm(e->cur, t, TCB_SCALE_ADD);
        prof_end(e);
        if (launched) return AVA_OK;
    }
    // with fast products a prompt chunk's k-WTA output is multiplied densely on the tensor cores as well (a quarter of
    // its entries are non-zero: over thousands of token-rows the dense product is the shorter one); a decode step's
    // few hundred rows keep the exact event sum
    if (sparse && e->fast && w.wt.p && M >= 1024) sparse = false;
    if (e->fast && !sparse && !row_gain && w.wt.p && lda == w.din && w.din % 64 == 0 && w.dout % 4 == 0) {
        const size_t need = (size_t)3 * M * w.din * sizeof(uint16_t);
        if (e->cur_w->limbs.bytes < need) {
            CK(e->cur_w->limbs.alloc(need));
            e->cur_w->limbs_src = nullptr;
        }
        if (!(e->cur_w->limbs_src == A && e->cur_w->limbs_rows == M)) {  // the producer did not leave them
            prof_begin(e, "tc.split3");
            launch_split3(e->cur, A, (int64_t)M * w.din, e->cur_w->limbs.as<uint16_t>());
            prof_end(e);
        }
        e->cur_w->limbs_src = nullptr;  // one product per set of limbs
        TcGemmArgs t{};
        t.a_limbs = e->cur_w->limbs.as<uint16_t>();
        t.w_bf16 = w.wt.as<uint16_t>();
        t.scale = w.sp();
        t.C = epi == EPI_LIF ? e->cur_w->yraw.as<float>() : C;  // the currents' buffer is free while the LIF layer runs
        t.ldc = epi == EPI_LIF ? w.dout : ldc;
        t.M = M;
        t.N = w.dout;
        t.K = w.din;
        t.status = e->status.as<uint32_t>();
        prof_begin(e, cls);
        const bool launched = launch_tc_gemm(e->cur, t, epi == EPI_LIF ? EPI_STORE : epi);
        prof_end(e);
        if (launched) {
            if (epi == EPI_LIF) {
                prof_begin(e, "lif");
                launch_lif(e->cur, e->cur_w->yraw.as<float>(), *lif, M, w.dout);
                prof_end(e);
            }
            return AVA_OK;
        }
    }
    prof_begin(e, cls);
    // the event sum takes the dense mix that follows it along (mix->streams is cleared to say so)
    const bool with_mix = mix && mix->streams && sparse && event_takes_mix(g, epi, mix->n_streams);
    const bool with_kw = mix && mix->kw_u;   // the k winners made inside the event kernel (a few rows): checked by the caller
    MixArgs pass;
    if (with_mix) pass = *mix;
    if (with_kw) { pass.kw_u = mix->kw_u; pass.kw_k = mix->kw_k; pass.kw_relu2 = mix->kw_relu2; }
    if (with_kw && !(sparse && event_small_covers(g, epi))) return e->fail(AVA_ERR_ARG, "the k winners inside the event sum: shape not covered");
    if (sparse && launch_q8_event(e->cur, g, epi, (with_mix || with_kw) ? &pass : nullptr)) {
        if (with_mix) mix->streams = nullptr;
    } else if (!(e->gemm2 && M > 16 && launch_q8_gemm2(e->cur, g, epi, e->sm_count))) {
        launch_q8_gemm(e->cur, g, epi, e->sm_count);
    }
    prof_end(e);
    return AVA_OK;
}

// T tokens per row (T = 1: the decode step), everything queued on the engine's stream.  tok is [T][rows] on the
// device; logits/next (device, may be null) get the LAST token's [rows, vocab] / [rows], or with all_logits every
// token's [T][rows][vocab].  With T > 1 the products, norms, gates and the MLP run over all T x rows token-rows at
// once, and the three recurrences walk the chunk in order inside their kernels: the LIF scan, the fast-weight pass
// with its slice resident in shared memory, the engram read token by token.  Every value is the one T single steps give.
enum StepPhase { PHASE_ALL = 0, PHASE_BEGIN = 1, PHASE_END = 2 };  // BEGIN stops once the engram's q,k,v exist; END resumes after its read

// whether a chunk of T tokens takes the chunk-parallel (tensor-core) form of the memory: then the state itself is worked on
bool chunk_form_applies(const ava_engine* e, int T) {
    return e->fast && e->chunk_mem && T > 1 && !e->keep && mem_chunk_covers(e->cfg.head_size, T, e->cfg.mem_momentum);
}


// One lane: rows [r0, r0 + rows) of the state, with the lane's work buffers, queued on stream st.  tok, logits and next
// are the caller's whole buffers (a lane reads and writes its own rows of them).
// blk0, blk1: the blocks [blk0, blk1) queued by this call (with what precedes block 0 when blk0 == 0, and the head and the
// host's bookkeeping when blk1 reaches the last block), so that a step's lanes can be queued block by block in turn.
int step_rows(ava_engine* e, Work& w, cudaStream_t st, ava_state* s, int r0, int rows, const uint32_t* tok, float* logits, uint32_t* next, bool want_logits,
              int T, bool all_logits, StepPhase phase, int blk0 = 0, int blk1 = 1 << 30) {
    const ava_config& c = e->cfg;
    const int d = c.d, L = c.n_blocks, nh = e->nh(), hs = c.head_size, H = c.hidden;
    e->cur = st;
    e->cur_w = &w;
    tok += r0;  // a lane other than the first exists only for T == 1: its tokens are rows r0.. of the one token
    const size_t Sd = (size_t)s->rows * d;  // one block's carried LIF state over ALL rows of the state
    const size_t so = (size_t)r0 * d;       // this lane's first row inside a block's state
    const int M = rows * T;  // token-rows, time-major: token t of row r is token-row t * rows + r
    float* x = w.x.as<float>();
    float* h = w.h.as<float>();
    float* streams = c.dense ? w.streams.as<float>() : nullptr;
    const size_t Md = (size_t)M * d;        // one activation buffer of the chunk
    const size_t Rd = (size_t)rows * d;     // one block's carried LIF state

    // the engram's capacity is checked on the host's mirror of the counts before anything moves
    int n_max = 0;
    if (c.eng_block >= 0 && phase == PHASE_ALL) {
        for (int r = r0; r < r0 + rows; ++r) {
            if (s->keep == s->ring && s->n_host[r] + T > s->ring)
                return e->fail(AVA_ERR_CAPACITY, "engram store of row %d is full (%d tokens)", r, s->ring);
            n_max = std::max(n_max, std::min(s->n_host[r] + T - 1, s->keep) + 1);
        }
    }

    const bool head_part = blk0 == 0, tail_part = blk1 >= L;
    if (phase != PHASE_END && head_part) {
        prof_begin(e, "embed");
        launch_embed(st, e->tok_emb.as<float>(), tok, M, d, c.vocab, x, streams, e->status.as<uint32_t>(), c.letters ? e->letters.as<float>() : nullptr);
        prof_end(e);
        dbg(e, "x_in", -1, x, M, d);
    }
    // TH: the relay reads the stream (16 numbers per token-row) into its sum and sets block j's gates; h and the gates'
    // scratch are free at both places it is called from
    auto relay_read = [&](int j) {
        prof_begin(e, "relay");
        launch_rmsnorm(st, x, e->ones.as<float>(), M, d, h);
        launch_chain_gemv(st, h, e->th_read.as<float>() + (size_t)j * d * 16, M, d, 16, e->gate_chunk, w.gz.as<float>());
        launch_relay(st, w.gz.as<float>(), w.th_acc.as<float>(), j == 0, j + 1, e->th_gate.as<float>() + (size_t)j * 32,
                     e->th_bias.as<float>() + (size_t)j * 2, M, w.th_g.as<float>());
        prof_end(e);
        e->launches += 2;
        dbg(e, "th_g", j, w.th_g.as<float>(), M, 4);
    };
    if (c.rhythm && phase != PHASE_END && head_part) {
        // Y: the clocks at every token of the chunk, from the input (after the letters): reset read-out, times, phase features
        prof_begin(e, "rhythm");
        launch_rmsnorm(st, x, e->ones.as<float>(), M, d, h);
        launch_chain_gemv(st, h, e->rhy_wr.as<float>(), M, d, 4, e->gate_chunk, w.gz.as<float>());
        launch_rhythm(st, w.gz.as<float>(), e->rhy_br.as<float>(), e->rhy_lw.as<float>(), rows, T, s->rh.as<float>() + (size_t)r0 * 2, w.rh_f.as<float>());
        prof_end(e);
        e->launches += 2;
        dbg(e, "rh_f", -1, w.rh_f.as<float>(), M, 4);
    }
    if (c.thalamus && phase != PHASE_END && head_part) relay_read(0);
    for (int i = std::max(phase == PHASE_END ? c.eng_block : 0, blk0); i < std::min(L, blk1); ++i) {
        BlockDev& b = *e->blocks[i];
        if (c.thalamus && !(phase == PHASE_END && i == c.eng_block))
            CK(cudaMemcpyAsync(w.x_in.p, x, Md * sizeof(float), cudaMemcpyDeviceToDevice, st));  // the residual rule's x_in
        const float* th_mem = c.thalamus ? w.th_g.as<float>() + 1 : nullptr;
        if (!(phase == PHASE_END && i == c.eng_block)) {
        // ---- the spiking memory
        // one sequence or a handful: the norm is taken inside the product that reads it (one kernel fewer per norm)
        const bool few = T == 1 && !e->fast && !e->keep && M <= gemv_max_rows();
        bool h_lif_fused = few && !(c.mood > 0 && i > 0);
        if (!h_lif_fused) {
        prof_begin(e, "rmsnorm");
        launch_rmsnorm(st, x, b.mem_norm.as<float>(), M, d, h, limbs_for(e, h, M, d));
        prof_end(e);
        }
        dbg(e, "h_lif", i, h, M, d);
        LifParams lp{};
        lp.beta = b.beta.as<float>();
        lp.theta = c.theta ? b.theta.as<float>() : nullptr;
        lp.rho = c.alif ? b.rho.as<float>() : nullptr;
        lp.gain = c.alif ? b.again.as<float>() : nullptr;
        lp.v = s->lif_v.as<float>() + (size_t)i * Sd + so;
        lp.s = s->lif_s.as<float>() + (size_t)i * Sd + so;
        lp.a = c.alif ? s->lif_a.as<float>() + (size_t)i * Sd + so : nullptr;
        lp.spikes = c.spikes;
        lp.lif_scale = c.lif_scale;
        const float* nm = (c.neuromod > 0 && i > 0) ? w.sig.as<float>() : nullptr;  // the nucleus's signals reach the later blocks
        lp.ne = nm;
        const float* spikes = lp.s;
        const float* cur_gain = nullptr;
        if (c.mood > 0 && i > 0) {
            // M: the current times 1 + tanh(mood G) per token-row and channel, after NE
            prof_begin(e, "mood");
            launch_mood_gain(st, w.mood_all.as<float>(), c.mood, b.mood_g.as<float>(), M, d, w.mood_gain.as<float>());
            prof_end(e);
            cur_gain = w.mood_gain.as<float>();
        }
        if (h_lif_fused) {
            GemvPro pn;
            pn.kind = PRO_RMS;
            pn.gain = b.mem_norm.as<float>();
            if (gemm(e, "gemm.win_lif", x, d, b.win, nullptr, 0, M, EPI_LIF, &lp, false, nullptr, false, &pn) != AVA_OK) {
                h_lif_fused = false;
                prof_begin(e, "rmsnorm");
                launch_rmsnorm(st, x, b.mem_norm.as<float>(), M, d, h, nullptr);
                prof_end(e);
            }
        }
        if (h_lif_fused) {
        } else if (T == 1 && !cur_gain) {
            gemm(e, "gemm.win_lif", h, d, b.win, nullptr, 0, M, EPI_LIF, &lp);
        } else {
            // currents of the whole chunk, then the scan in time (buffers free at this point of the block are borrowed)
            gemm(e, "gemm.win", h, d, b.win, w.yraw.as<float>(), d, M, EPI_STORE);
            prof_begin(e, "lif_scan");
            launch_lif_scan(st, w.yraw.as<float>(), lp, rows, d, T, w.eo.as<float>(), cur_gain);
            prof_end(e);
            spikes = w.eo.as<float>();
        }
        dbg(e, "spikes", i, spikes, M, d);
        if (c.stp) {
            // the LIF keeps its spikes; what reaches W_out goes through the short-term-plastic synapse
            prof_begin(e, "stp");
            launch_stp(st, spikes, b.stp_U.as<float>(), b.stp_F.as<float>(), b.stp_D.as<float>(), b.stp_mix.as<float>(),
                       s->stp_u.as<float>() + (size_t)i * Sd + so, s->stp_x.as<float>() + (size_t)i * Sd + so, rows, d, T, w.eo.as<float>());
            prof_end(e);
            spikes = w.eo.as<float>();
            dbg(e, "stp_out", i, spikes, M, d);
        }
        gemm(e, "gemm.wout", spikes, d, b.wout, x, d, M, EPI_ADD, nullptr, true, nullptr, !c.stp);
        dbg(e, "x_lif", i, x, M, d);

        // ---- the fast-weight memory (kinds D and A; a kind-S block goes on to its MLP)
        if (c.fast_mem) {
        const int pw = e->proj_w();
        // one sequence or a handful: the norm in front of q|k|v|e|g and the gates is taken by both of its readers
        // themselves (each while its weights arrive), so it needs no kernel of its own
        GemvPro hebb_pro;
        hebb_pro.kind = PRO_RMS;
        hebb_pro.gain = b.hebb_norm.as<float>();
        bool norm_inside = false;
        if (few) {
            GemmArgs gq{};
            gq.A = x; gq.lda = d; gq.W = b.proj.qp(); gq.ldw = b.proj.dout; gq.M = M; gq.N = b.proj.dout; gq.K = b.proj.din; gq.ldc = pw;
            norm_inside = b.proj.din == d && q8_gemv_pro_covers(gq, hebb_pro) && gate_z_few_covers(x, b.gate_w.as<float>(), M, d, e->gate_cols) &&
                          !(reinterpret_cast<uintptr_t>(hebb_pro.gain) & 15);
        }
        if (!norm_inside) {
        prof_begin(e, "rmsnorm");
        launch_rmsnorm(st, x, b.hebb_norm.as<float>(), M, d, h, limbs_for(e, h, M, d));
        prof_end(e);
        }
        dbg(e, "h_mem", i, h, M, d);
        MemPrepArgs mp{};
        mp.h = norm_inside ? x : h;
        mp.h_gain = norm_inside ? hebb_pro.gain : nullptr;
        mp.proj = w.proj.as<float>();
        mp.ldp = pw;
        mp.gate_w = b.gate_w.as<float>(); mp.gate_cols = e->gate_cols; mp.gate_chunk = e->gate_chunk;
        mp.z = w.gz.as<float>(); mp.lra = w.lra.as<float>(); mp.lrb = w.lrb.as<float>();
        mp.ba = b.ba.as<float>(); mp.bb = b.bb.as<float>(); mp.wa2 = b.wa2.as<float>(); mp.wb2 = b.wb2.as<float>();
        mp.off = b.off.as<float>();
        mp.vres = (c.value_residual && i > 0 && b.vres.p) ? b.vres.as<float>() : nullptr;
        mp.v_first = w.v_first.as<float>();
        mp.first = c.value_residual && i == 0;
        mp.M = M; mp.d = d; mp.hs = hs; mp.rank = c.gate_rank;
        mp.e = w.ve.as<float>(); mp.v = w.vv.as<float>(); mp.w = w.vw.as<float>(); mp.ah = w.vah.as<float>();
        mp.qg = w.vqg.as<float>(); mp.ex = w.vex.as<float>(); mp.qw = w.qw.as<float>(); mp.qa = w.qa.as<float>();
        mp.qs = c.mem_momentum > 0.0f ? w.vqs.as<float>() : nullptr;
        mp.mom = c.mem_momentum;
        mp.fast = e->fast && !e->keep;
        // One token of the plain memory takes the streaming pass: this token's alpha, w, ah and values go straight into
        // the state's pending set (the one this step writes), the pass reads the set the step before wrote.
        const bool stream = T == 1 && !(c.mem_momentum > 0.0f);
        const bool stream_chunk = T > 1 && !(c.mem_momentum > 0.0f) && !chunk_form_applies(e, T);
        const int wset = s->pend_set ^ 1;
        if (stream) {
            mp.ex = s->pend_at(wset, 0, i) + so; mp.w = s->pend_at(wset, 1, i) + so; mp.ah = s->pend_at(wset, 2, i) + so; mp.v = s->pend_at(wset, 3, i) + so;
        }
        if (c.rhythm) {
            prof_begin(e, "rhythm");
            launch_rhythm_gates(st, w.rh_f.as<float>(), b.rh_w.as<float>(), b.rh_r.as<float>(), M, nh, w.rh_gw.as<float>(), w.rh_gr.as<float>());
            prof_end(e);
            mp.rh_w = w.rh_gw.as<float>();
        }
        const bool use_chunk = chunk_form_applies(e, T);
        if (use_chunk) {
            const size_t need = mem_chunk_workspace_bytes(rows * nh, hs, T / 64);
            if (w.chunk_ws.bytes < need) CK(w.chunk_ws.alloc(need));
            if (w.vqn.bytes < Md * sizeof(float)) { CK(w.vqn.alloc(Md * sizeof(float))); CK(w.vla.alloc(Md * sizeof(float))); }
            if (!w.chunk_flag.p) CK(w.chunk_flag.alloc(2 * sizeof(uint32_t)));
            mp.qn_out = w.vqn.as<float>();
            mp.la_out = w.vla.as<float>();
        }
        mp.ach = (c.neuromod > 0 && i > 0) ? w.sig.as<float>() + 1 : nullptr;
        mp.ach_stride = 4;
        mp.status = e->status.as<uint32_t>();
        if (e->keep) {
            if (w.side.bytes < Md * sizeof(float)) CK(w.side.alloc(Md * sizeof(float)));
            mp.be_out = w.side.as<float>();
        }
        // the gates' two projection stages read the normed input alone: on the lane's side stream they run beside the
        // q|k|v|e|g product (both are short of warps on their own); the per-row kernel then needs both
        // with fast products the first stage is a product of limbs on the tensor cores (the norm has left the limbs of h)
        bool tc_gates = false;
        if (e->fast && !e->keep && b.gate_wl.p && M % 128 == 0 && d % 64 == 0 && e->cur_w->limbs_src == h && e->cur_w->limbs_rows == M) {
            TcbArgs g{};
            g.a = e->cur_w->limbs.as<uint16_t>(); g.rows_a = M; g.b = b.gate_wl.as<uint16_t>(); g.rows_b = e->gate_cols;
            g.C = mp.z; g.ldc = e->gate_cols; g.c_batch_stride = 0; g.M = M; g.N = e->gate_cols; g.K = d; g.batch = 1;
            g.status = e->status.as<uint32_t>();
            prof_begin(e, "gate_z");
            tc_gates = launch_tc_bgemm(st, g, TCB_STORE);
            prof_end(e);
            if (tc_gates) {
                launch_mem_gates_low(st, mp);
                e->launches++;
            }
        }
        const bool fork = !tc_gates && w.side_stream != nullptr && (!e->prof || e->prof_lanes) && !e->keep;
        if (fork) {
            CK(cudaEventRecord(w.side_go, st));
            CK(cudaStreamWaitEvent(w.side_stream, w.side_go, 0));
            launch_mem_gates(w.side_stream, mp);
            CK(cudaEventRecord(w.side_done, w.side_stream));
        }
        if (norm_inside) {
            const int prc = gemm(e, "gemm.qkveg", x, d, b.proj, w.proj.as<float>(), pw, M, EPI_STORE, nullptr, false, nullptr, false, &hebb_pro);
            if (prc != AVA_OK) return e->fail(AVA_ERR_CUDA, "the q|k|v|e|g product with its norm inside was refused after it had been accepted");
        } else {
            gemm(e, "gemm.qkveg", h, d, b.proj, w.proj.as<float>(), pw, M, EPI_STORE);
        }
        dbg(e, "qkveg", i, w.proj.as<float>(), M, pw);
        prof_begin(e, "mem_prep");
        if (tc_gates) {
            launch_mem_prep_rows(st, mp);
            e->launches -= 2;  // counted where they were queued
        } else if (fork) {
            CK(cudaStreamWaitEvent(st, w.side_done, 0));
            launch_mem_prep_rows(st, mp);
        } else {
            launch_mem_prep(st, mp);
        }
        prof_end(e);
        if (e->keep) dbg(e, "be", i, w.side.as<float>(), M, d);
        e->launches += 2;  // the two stages of the gate projections before it
        dbg(e, "ek", i, mp.e, M, d); dbg(e, "v", i, mp.v, M, d); dbg(e, "w", i, mp.w, M, d); dbg(e, "ah", i, mp.ah, M, d);
        dbg(e, "qg", i, mp.qg, M, d); dbg(e, "ex", i, mp.ex, M, d); dbg(e, "qw", i, mp.qw, M, nh); dbg(e, "qa", i, mp.qa, M, nh);
        MemHeadsArgs mh{};
        mh.f = s->mem_f.as<float>() + ((size_t)i * Sd + so) * hs;
        mh.s = c.mem_momentum > 0.0f ? s->mem_s.as<float>() + ((size_t)i * Sd + so) * hs : nullptr;
        mh.qs = mp.qs;
        mh.mom = c.mem_momentum;
        mh.M = rows; mh.nh = nh; mh.hs = hs; mh.cw = e->cw; mh.chunk_rows = e->rb;
        mh.e = mp.e; mh.v = mp.v; mh.w = mp.w; mh.ah = mp.ah; mh.qg = mp.qg; mh.ex = mp.ex; mh.qw = mp.qw; mh.qa = mp.qa;
        mh.y = w.yraw.as<float>();
        mh.status = e->status.as<uint32_t>();
        prof_begin(e, "mem_heads");
        bool chunked = false;
        if (use_chunk) {
            // the tolerance mode reads a prompt's chunk with the chunk-parallel form on the tensor cores, unless the
            // rates of some 64 tokens forget too fast for it (then the token loop below, for this block and chunk)
            ChunkArgs ca{};
            ca.HB = rows * nh; ca.hs = hs; ca.nC = T / 64; ca.cw = e->cw; ca.tok_stride = (int64_t)rows * d;
            ca.qn = mp.qn_out; ca.e = mp.e; ca.w = mp.w; ca.ah = mp.ah; ca.v = mp.v; ca.la = mp.la_out; ca.y = mh.y; ca.F = mh.f;
            ca.flags = w.chunk_flag.as<uint32_t>(); ca.status = e->status.as<uint32_t>();
            mem_chunk_carve(ca, w.chunk_ws.p);
            CK(cudaMemsetAsync(ca.flags, 0, sizeof(uint32_t), st));
            launch_mem_chunk_scale(st, ca);
            uint32_t out_of_range = 0;
            CK(cudaMemcpyAsync(&out_of_range, ca.flags, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
            CK(cudaStreamSynchronize(st));
            e->launches += 3;
            if (!(out_of_range & 1u)) {
                if (!launch_mem_chunk_rest(st, ca)) return e->fail(AVA_ERR_CUDA, "chunk-parallel memory: a launch was refused");
                e->launches += mem_chunk_launches(ca.nC) - 4;
                chunked = true;
                ++e->chunked_blocks;
            } else {
                ++e->chunk_fallbacks;
            }
        }
        if (chunked) {
        } else if (stream_chunk) {
            // a chunk of tokens, one streaming pass per token: token t's pass applies token t - 1's update (the vectors
            // of the whole chunk lie in the work buffers; the first token takes what the state has pending) and leaves
            // its own rr beside them; the last token's update stays pending in the state.  One read and one write of
            // the state per token, as in decoding; the same bits.
            if (w.vrr.bytes < Md * sizeof(float)) CK(w.vrr.alloc(Md * sizeof(float)));
            for (int t = 0; t < T; ++t) {
                const size_t at = (size_t)t * Rd, ah_ = (size_t)t * rows * nh;
                MemStreamArgs ms{};
                ms.f = mh.f; ms.M = rows; ms.nh = nh; ms.hs = hs; ms.cw = e->cw;
                ms.e = mp.e + at; ms.qg = mp.qg + at; ms.v = mp.v + at; ms.qw = mp.qw + ah_; ms.qa = mp.qa + ah_;
                ms.y = mh.y + at;
                ms.rr_out = w.vrr.as<float>() + at;
                if (t > 0) {
                    const size_t pr = at - Rd;
                    ms.px = mp.ex + pr; ms.pw = mp.w + pr; ms.pah = mp.ah + pr; ms.pv = mp.v + pr; ms.prr = w.vrr.as<float>() + pr;
                } else if (s->pending) {
                    const int rset = s->pend_set;
                    ms.px = s->pend_at(rset, 0, i) + so; ms.pw = s->pend_at(rset, 1, i) + so; ms.pah = s->pend_at(rset, 2, i) + so;
                    ms.pv = s->pend_at(rset, 3, i) + so; ms.prr = s->pend_at(rset, 4, i) + so;
                }
                if (!launch_mem_stream(st, ms)) return e->fail(AVA_ERR_CAPACITY, "memory head size not covered by the streaming pass");
            }
            const size_t last = (size_t)(T - 1) * Rd;
            const float* srcs[5] = {mp.ex + last, mp.w + last, mp.ah + last, mp.v + last, w.vrr.as<float>() + last};
            for (int k = 0; k < 5; ++k)
                CK(cudaMemcpyAsync(s->pend_at(wset, k, i) + so, srcs[k], Rd * sizeof(float), cudaMemcpyDeviceToDevice, st));
            e->launches += T - 1;
        } else if (stream) {
            MemStreamArgs ms{};
            ms.f = mh.f; ms.M = rows; ms.nh = nh; ms.hs = hs; ms.cw = e->cw;
            if (s->txn_pingpong && s->pending) ms.f_out = s->mem_f_alt.as<float>() + ((size_t)i * Sd + so) * hs;
            ms.early_state = 1;   // the kernel queued just before (the gates' per-row part) does not write the state
            ms.e = mp.e; ms.qg = mp.qg; ms.v = mp.v; ms.qw = mp.qw; ms.qa = mp.qa;
            ms.y = mh.y;
            ms.rr_out = s->pend_at(wset, 4, i) + so;
            if (s->pending) {
                const int rset = s->pend_set;
                ms.px = s->pend_at(rset, 0, i) + so; ms.pw = s->pend_at(rset, 1, i) + so; ms.pah = s->pend_at(rset, 2, i) + so;
                ms.pv = s->pend_at(rset, 3, i) + so; ms.prr = s->pend_at(rset, 4, i) + so;
            }
            if (!launch_mem_stream(st, ms)) return e->fail(AVA_ERR_CAPACITY, "memory head size not covered by the streaming pass");
        } else {
            launch_mem_heads_seq(st, mh, T);
        }
        prof_end(e);
        dbg(e, "y_raw", i, mh.y, M, d);
        bool post_fused = false;
        if (few && !c.dendrite && !c.rhythm) {
            GemvPro pp;
            pp.kind = PRO_POST;
            pp.gate = c.out_gate ? w.proj.as<float>() + 4 * d : nullptr;
            pp.ldg = pw;
            pp.hs = hs;
            post_fused = gemm(e, "gemm.wo", mh.y, d, b.wo, x, d, M, EPI_ADD, nullptr, false, th_mem, false, &pp) == AVA_OK;
        }
        if (!post_fused) {
        prof_begin(e, "mem_post");
        launch_mem_post(st, mh.y, c.out_gate ? w.proj.as<float>() + 4 * d : nullptr, pw, M, d, hs, w.y.as<float>(), limbs_for(e, w.y.as<float>(), M, d),
                        c.rhythm ? w.rh_gr.as<float>() : nullptr);
        prof_end(e);
        }
        dbg(e, "y", i, w.y.as<float>(), M, d);
        if (post_fused) {
        } else if (c.dendrite) {
            // P: the read after W_o is kept, the context of this block's dendrites
            gemm(e, "gemm.wo", w.y.as<float>(), d, b.wo, w.ctx.as<float>(), d, M, EPI_STORE);
            prof_begin(e, "add");
            launch_add_into(st, x, w.ctx.as<float>(), (int64_t)Md, th_mem, d);
            prof_end(e);
        } else {
            gemm(e, "gemm.wo", w.y.as<float>(), d, b.wo, x, d, M, EPI_ADD, nullptr, false, th_mem);
        }
        dbg(e, "x_mem", i, x, M, d);
        }
        }

        // ---- the engram
        if (i == c.eng_block) {
            if (phase != PHASE_END) {
                bool eng_fused = false;
                if (T == 1 && !e->fast && !e->keep && M <= gemv_max_rows()) {
                    GemvPro pn;
                    pn.kind = PRO_RMS;
                    pn.gain = b.eng_norm.as<float>();
                    eng_fused = gemm(e, "gemm.eng_qkv", x, d, b.eqkv, w.eqkv.as<float>(), 3 * d, M, EPI_STORE, nullptr, false, nullptr, false, &pn) == AVA_OK;
                }
                if (!eng_fused) {
                prof_begin(e, "rmsnorm");
                launch_rmsnorm(st, x, b.eng_norm.as<float>(), M, d, h, limbs_for(e, h, M, d));
                prof_end(e);
                gemm(e, "gemm.eng_qkv", h, d, b.eqkv, w.eqkv.as<float>(), 3 * d, M, EPI_STORE);
                }
                dbg(e, "eng_qkv", i, w.eqkv.as<float>(), M, 3 * d);
            }
            if (phase == PHASE_BEGIN) {
                cudaError_t le0 = take_launch_error();
                if (le0 == cudaSuccess) le0 = cudaGetLastError();
                if (le0 != cudaSuccess) return e->cuda_fail(le0, "kernel launch");
                return AVA_OK;
            }
            EngramArgs ea{};
            ea.qkv = w.eqkv.as<float>();
            const size_t kv_row = (size_t)d * s->ring * s->kv_elem();  // bytes of one row's keys (or values): [heads][ring][hs]
            ea.k = (char*)s->eng_k.p + r0 * kv_row; ea.v = (char*)s->eng_v.p + r0 * kv_row;
            ea.n = s->eng_n.as<int32_t>() + r0; ea.start = s->eng_start.as<int32_t>() + r0;
            ea.M = rows; ea.d = d; ea.hs = c.eng_head_size; ea.cap = s->ring; ea.keep = s->keep; ea.bf16 = c.eng_store_bf16;
            ea.status = e->status.as<uint32_t>();
            // the read is causal: token t sees the store as tokens 0..t left it, so the chunk goes token by token.  A
            // store that one block's shared memory can hold is read in one pass (the reference's order, bit for bit);
            // a longer one, or any store when the segmented read is switched on, in segments merged afterwards.
            const int enh = d / c.eng_head_size;
            const bool segmented = e->long_seg > 0 || !engram_fits_one_block(d, c.eng_head_size, n_max);
            const int seg_len = e->long_seg > 0 ? e->long_seg : 2048;
            const int n_seg = engram_segments(n_max, seg_len);
            if (segmented) {
                const size_t need = (size_t)rows * enh * n_seg * (2 + c.eng_head_size) * sizeof(float);
                if (w.eng_partial.bytes < need) CK(w.eng_partial.alloc(need));
            }
            // the tolerance mode reads a prompt chunk in one causal pass on the tensor cores, when the store neither wraps
            // nor trims inside the chunk (head size 64, bf16 store)
            bool chunk_read = e->fast && e->chunk_mem && T > 1 && phase == PHASE_ALL && !e->keep && c.eng_store_bf16 && c.eng_head_size == 64 &&
                              s->keep == s->ring;
            for (int r = r0; r < r0 + rows && chunk_read; ++r) chunk_read = s->start_host[r] + s->n_host[r] + T <= s->ring;
            if (chunk_read) {
                EngramChunkArgs ca{};
                ca.qkv = w.eqkv.as<float>(); ca.o = w.eo.as<float>(); ca.k = ea.k; ca.v = ea.v; ca.n = ea.n; ca.start = ea.start;
                ca.M = rows; ca.d = d; ca.hs = c.eng_head_size; ca.cap = s->ring; ca.T = T; ca.bf16 = 1; ca.status = ea.status;
                prof_begin(e, "engram.chunk");
                chunk_read = launch_engram_chunk(st, ca);
                prof_end(e);
                if (chunk_read) {
                    e->launches += 2;
                    ++e->chunked_reads;
                }
            }
            for (int t = 0; t < T && phase == PHASE_ALL && !chunk_read; ++t) {
                ea.qkv = w.eqkv.as<float>() + (size_t)t * rows * 3 * d;
                ea.o = w.eo.as<float>() + (size_t)t * Rd;
                if (!segmented) {
                    prof_begin(e, "engram");
                    if (!launch_engram(st, ea, n_max))
                        return e->fail(AVA_ERR_CAPACITY, "engram read over %d tokens does not fit this kernel's shared memory", n_max);
                    prof_end(e);
                    e->launches++;  // the small kernel that moves the counts on
                } else {
                    prof_begin(e, "engram.append");
                    launch_engram_append(st, ea);
                    prof_end(e);
                    prof_begin(e, "engram.partial");
                    if (!launch_engram_partial(st, ea, seg_len, n_seg, w.eng_partial.as<float>()))
                        return e->fail(AVA_ERR_CAPACITY, "engram segments of %d keys do not fit shared memory", seg_len);
                    prof_end(e);
                    prof_begin(e, "engram.combine");
                    launch_engram_combine(st, w.eng_partial.as<float>(), rows, enh, c.eng_head_size, n_seg, ea.o);
                    prof_end(e);
                    launch_engram_trim(st, ea);
                    e->launches += 2;
                }
            }
            ea.o = w.eo.as<float>();
            dbg(e, "eng_o", i, ea.o, M, d);
            if (e->keep) {
                // the read as it is added (the token trace shows it): the same product stored, then the same addition
                if (w.side.bytes < Md * sizeof(float)) CK(w.side.alloc(Md * sizeof(float)));
                gemm(e, "gemm.eng_wo", ea.o, d, b.ewo, w.side.as<float>(), d, M, EPI_STORE);
                dbg(e, "eng_r", i, w.side.as<float>(), M, d);
                launch_add_into(st, x, w.side.as<float>(), (int64_t)Md);
            } else {
                gemm(e, "gemm.eng_wo", ea.o, d, b.ewo, x, d, M, EPI_ADD);
            }
            dbg(e, "x_eng", i, x, M, d);
        }

        // ---- the sparse MLP
        bool mlp_fused = false;
        if (T == 1 && !e->fast && !e->keep && M <= gemv_max_rows()) {
            GemvPro pn;
            pn.kind = PRO_RMS;
            pn.gain = b.mlp_norm.as<float>();
            mlp_fused = gemm(e, "gemm.w1", x, d, b.w1, w.u.as<float>(), H, M, EPI_STORE, nullptr, false, nullptr, false, &pn) == AVA_OK;
        }
        if (!mlp_fused) {
        prof_begin(e, "rmsnorm");
        launch_rmsnorm(st, x, b.mlp_norm.as<float>(), M, d, h, limbs_for(e, h, M, d));
        prof_end(e);
        gemm(e, "gemm.w1", h, d, b.w1, w.u.as<float>(), H, M, EPI_STORE);
        }
        dbg(e, "u", i, w.u.as<float>(), M, H);
        // one sequence or a handful: W2's event kernel makes the k winners itself (each of its blocks selects them from
        // the 3072 pre-activations while nothing else runs anyway), so they need no kernel of their own
        bool kw_inside = false;
        if (T == 1 && !e->fast && !e->keep && !c.dendrite && !(c.dopamine && i > 0) && M <= gemv_max_rows()) {
            GemmArgs gq{};
            gq.W = b.w2.qp(); gq.ldw = b.w2.dout; gq.M = M; gq.N = b.w2.dout; gq.K = b.w2.din; gq.ldc = d;
            kw_inside = event_small_covers(gq, EPI_ADD);
        }
        if (!kw_inside) {
        prof_begin(e, "kwta");
        // a prompt chunk in the tolerance mode multiplies the k-WTA's output densely on the tensor cores: its limbs are made here
        launch_kwta(st, w.u.as<float>(), M, H, c.kwta_k, c.relu2, w.act.as<float>(),
                    (M >= 1024 && b.w2.wt.p && !c.dendrite) ? limbs_for(e, w.act.as<float>(), M, H) : nullptr);
        prof_end(e);
        }
        dbg(e, "a", i, w.act.as<float>(), M, H);
        if (c.dendrite && c.fast_mem) {
            // P: the units times 1 + tanh(head_norm(ctx) A B); h is free here
            prof_begin(e, "dendrite");
            launch_rmsnorm(st, w.ctx.as<float>(), e->ones.as<float>(), M, d, h);
            launch_chain_gemv(st, h, b.dend_a.as<float>(), M, d, 32, e->gate_chunk, w.dz1.as<float>());
            launch_dend_gain(st, w.dz1.as<float>(), 32, b.dend_b.as<float>(), M, H, w.act.as<float>());
            prof_end(e);
            e->launches += 2;
            dbg(e, "a_dend", i, w.act.as<float>(), M, H);
        }
        const float* nm_da = (c.neuromod > 0 && i > 0) ? w.sig.as<float>() + 2 : nullptr;
        MixArgs mixa;   // W2's event sum takes the dense mix along in its epilogue (one kernel fewer in the block's chain)
        if (c.dense && !c.thalamus && !e->fast && !e->keep) {
            mixa.streams = streams;
            mixa.w = b.dense.as<float>();
            mixa.n_streams = i + 2;
        }
        const bool mix_asked = mixa.streams != nullptr;
        if (kw_inside) {
            mixa.kw_u = w.u.as<float>();
            mixa.kw_k = c.kwta_k;
            mixa.kw_relu2 = c.relu2;
        }
        if (c.dopamine && i > 0) {
            // DA: the MLP's output times 1 + tanh(z w + c), z the token's surprise / ln V, before the nucleus's DA signal
            gemm(e, "gemm.w2", w.act.as<float>(), H, b.w2, w.y2.as<float>(), d, M, EPI_STORE, nullptr, true);
            prof_begin(e, "dopamine");
            launch_da_add(st, x, w.y2.as<float>(), w.sur_z.as<float>(), b.da_w.as<float>(), b.da_c.as<float>(), nm_da, M, d);
            prof_end(e);
        } else {
            gemm(e, "gemm.w2", w.act.as<float>(), H, b.w2, x, d, M, EPI_ADD, nullptr, true, nm_da, false, nullptr, &mixa);
        }
        if (c.thalamus) {
            prof_begin(e, "relay");
            launch_relay_res(st, x, w.x_in.as<float>(), w.th_g.as<float>(), M, d);
            prof_end(e);
        }
        if (c.dense && !(mix_asked && !mixa.streams)) {
            prof_begin(e, "dense_mix");
            launch_dense_mix(st, x, streams, b.dense.as<float>(), i + 2, (int64_t)Md);
            prof_end(e);
        }
        dbg(e, "x_out", i, x, M, d);
        if (c.thalamus && i + 1 < L) relay_read(i + 1);
        if (i == 0 && (c.dopamine || c.mood > 0)) {
            // DA / M: the surprise at each token, from the head's logits for block 0's normed output at the position before
            // it (the carried one for a chunk's first token), then the mood's scan; the carried values move on
            prof_begin(e, "surprise");
            launch_rmsnorm(st, x, e->final_norm.as<float>(), M, d, w.sur_xf.as<float>());
            CK(cudaMemcpyAsync(w.sur_in.p, s->sur_prev.as<float>() + so, Rd * sizeof(float), cudaMemcpyDeviceToDevice, st));
            if (T > 1)
                CK(cudaMemcpyAsync(w.sur_in.as<float>() + Rd, w.sur_xf.p, (size_t)(T - 1) * Rd * sizeof(float), cudaMemcpyDeviceToDevice, st));
            prof_end(e);
            gemm(e, "gemm.sur_head", w.sur_in.as<float>(), d, e->head, w.sur_logits.as<float>(), c.vocab, M, EPI_STORE);
            prof_begin(e, "surprise");
            if (!launch_surprise(st, w.sur_logits.as<float>(), c.vocab, tok, s->sur_valid.as<float>() + r0, rows, T, w.sur_s.as<float>(), w.sur_z.as<float>()))
                return e->fail(AVA_ERR_CAPACITY, "the surprise kernel holds a vocabulary of up to 56320 in shared memory");
            if (c.mood > 0)
                launch_mood(st, w.sur_z.as<float>(), rows, T, c.mood, e->mood_lam.as<float>(), e->mood_win.as<float>(), e->mood_bin.as<float>(),
                            s->mood.as<float>() + (size_t)r0 * c.mood, w.mood_all.as<float>());
            CK(cudaMemcpyAsync(s->sur_prev.as<float>() + so, w.sur_xf.as<float>() + (size_t)(T - 1) * Rd, Rd * sizeof(float), cudaMemcpyDeviceToDevice, st));
            CK(cudaMemcpyAsync(s->sur_last.as<float>() + r0, w.sur_s.as<float>() + (size_t)(T - 1) * rows, rows * sizeof(float), cudaMemcpyDeviceToDevice, st));
            launch_fill(st, s->sur_valid.as<float>() + r0, rows, 1.0f);
            prof_end(e);
            e->launches += 3;
            dbg(e, "sur_z", 0, w.sur_z.as<float>(), M, 1);
        }
        if (i == 0 && c.neuromod > 0) {
            // the nucleus reads block 0's output: 2 sigmoid(rmsnorm(x, g) W + b) per token-row (h and the gates' scratch are free)
            prof_begin(e, "nucleus");
            launch_rmsnorm(st, x, e->nm_norm.as<float>(), M, d, h);
            launch_chain_gemv(st, h, e->nm_wn.as<float>(), M, d, 4, e->gate_chunk, w.gz.as<float>());
            launch_nucleus(st, w.gz.as<float>(), e->nm_bn.as<float>(), c.neuromod, M, w.sig.as<float>());
            prof_end(e);
            e->launches += 2;
            dbg(e, "nm_sig", 0, w.sig.as<float>(), M, 4);
        }
    }
    if (!tail_part) {
        cudaError_t le = take_launch_error();
        if (le == cudaSuccess) le = cudaGetLastError();
        if (le != cudaSuccess) return e->cuda_fail(le, "kernel launch");
        return AVA_OK;
    }
    if (want_logits || next) {
        // the head reads the last token's rows only, unless every position's logits were asked for
        const int first_row = all_logits ? 0 : (T - 1) * rows, head_rows = all_logits ? M : rows;
        float* lg = (logits ? logits : e->logits.as<float>()) + (size_t)r0 * c.vocab;
        bool head_fused = false;
        if (T == 1 && !e->fast && !e->keep && c.cb_units == 0 && head_rows <= gemv_max_rows()) {
            GemvPro pn;
            pn.kind = PRO_RMS;
            pn.gain = e->final_norm.as<float>();
            head_fused = gemm(e, "gemm.head", x + (size_t)first_row * d, d, e->head, lg, c.vocab, head_rows, EPI_STORE, nullptr, false, nullptr, false, &pn) == AVA_OK;
        }
        if (!head_fused) {
        prof_begin(e, "rmsnorm");
        launch_rmsnorm(st, x + (size_t)first_row * d, e->final_norm.as<float>(), head_rows, d, h, c.cb_units > 0 ? nullptr : limbs_for(e, h, head_rows, d));
        prof_end(e);
        }
        dbg(e, "x_final", -1, h, head_rows, d);
        if (c.cb_units > 0) {
            // CB: the final normed state plus the read-out of the sparse code of it and the token's embedding
            const int G = c.cb_units;
            prof_begin(e, "cerebellum");
            launch_cb_inputs(st, e->tok_emb.as<float>(), tok + first_row, head_rows, d, c.vocab, w.cb_emb.as<float>());
            launch_rmsnorm(st, w.cb_emb.as<float>(), e->ones.as<float>(), head_rows, d, w.cb_en.as<float>());
            launch_cb_units(st, h, w.cb_en.as<float>(), e->cb_idx.as<uint32_t>(), e->cb_sgn.as<float>(), G, d, head_rows, w.cb_h.as<float>());
            launch_kwta(st, w.cb_h.as<float>(), head_rows, G, G / 32, 0, w.cb_a.as<float>());
            launch_cb_read(st, w.cb_a.as<float>(), G, w.cb_lj.as<int>(), w.cb_lc.as<float>(), w.cb_n.as<int>(), e->cb_w.as<float>(), head_rows, d, h);
            prof_end(e);
            e->launches += 5;
            dbg(e, "x_cb", -1, h, head_rows, d);
        }
        if (next) next += r0;
        if (!head_fused) gemm(e, "gemm.head", h, d, e->head, lg, c.vocab, head_rows, EPI_STORE);
        if (next) {
            prof_begin(e, "argmax");
            launch_argmax(st, lg + (all_logits ? (size_t)(T - 1) * rows * c.vocab : 0), rows, c.vocab, next);
            prof_end(e);
        }
    }
    // the host's mirror of the engram counts moves as the kernels move them
    if (c.eng_block >= 0 && phase == PHASE_ALL)
        for (int r = r0; r < r0 + rows; ++r)
            for (int t = 0; t < T; ++t) {
                const int n = s->n_host[r] + 1;
                if (n > s->keep) {
                    s->start_host[r] = (s->start_host[r] + (n - s->keep)) % s->ring;
                    s->n_host[r] = s->keep;
                } else {
                    s->n_host[r] = n;
                }
            }
    for (int r = r0; r < r0 + rows; ++r) s->seen[r] += T;
    cudaError_t le = take_launch_error();
    if (le == cudaSuccess) le = cudaGetLastError();
    if (le != cudaSuccess) return e->cuda_fail(le, "kernel launch");
    return AVA_OK;
}

int flush_pending(ava_engine* e, ava_state* s);

// The step of a whole state.  A decode step (T == 1) of enough rows runs as `n_lanes` lanes: contiguous windows of the
// rows, each with its own work buffers and stream, forked from the engine's stream and joined back into it, so callers
// see one stream as before.  Rows are independent (src/state.rs:13-15), so the lanes compute the same bits.
int step_device(ava_engine* e, ava_state* s, const uint32_t* tok, float* logits, uint32_t* next, bool want_logits, int T = 1, bool all_logits = false,
                StepPhase phase = PHASE_ALL) {
    // a token's pending set is complete once its last block is through: a step split in two (BEGIN, END) writes one set
    // across both halves, so the sets change places after ALL or END only
    // (a chunk of tokens of the plain memory streams too, token after token, unless it takes the chunk-parallel form)
    const bool streams_state = e->cfg.fast_mem && !(e->cfg.mem_momentum > 0.0f) && phase != PHASE_BEGIN && !(T > 1 && chunk_form_applies(e, T));
    if (!streams_state && T > 1) {
        const int frc = flush_pending(e, s);  // a chunk of tokens works on the state itself
        if (frc) return frc;
    }
    int lanes = 1;
    // (with fast products lanes measured no gain: 4.52 ms per step either way, so that mode keeps one lane)
    if (e->n_lanes > 1 && T == 1 && phase == PHASE_ALL && !e->keep && !e->fast && (!e->prof || e->prof_lanes))
        lanes = std::max(1, std::min(e->n_lanes, s->rows / 48));  // a lane of fewer rows gains nothing
    if (lanes == 1) {
        const int rc1 = step_rows(e, *e, e->stream, s, 0, s->rows, tok, logits, next, want_logits, T, all_logits, phase);
        if (rc1 == AVA_OK && streams_state) {
            s->pend_set ^= 1;
            s->pending = true;
        }
        return rc1;
    }
    const int per = (s->rows + lanes - 1) / lanes;
    while ((int)e->more_lanes.size() < lanes - 1) {
        std::unique_ptr<Work> w(new Work());
        CK(cudaStreamCreateWithFlags(&w->lane_stream, cudaStreamNonBlocking));
        CK(cudaEventCreateWithFlags(&w->lane_done, cudaEventDisableTiming));
        if (e->side_stream) {
            CK(cudaStreamCreateWithFlags(&w->side_stream, cudaStreamNonBlocking));
            CK(cudaEventCreateWithFlags(&w->side_go, cudaEventDisableTiming));
            CK(cudaEventCreateWithFlags(&w->side_done, cudaEventDisableTiming));
        }
        e->more_lanes.push_back(std::move(w));
    }
    if (!e->fork_ev) CK(cudaEventCreateWithFlags(&e->fork_ev, cudaEventDisableTiming));
    for (int l = 1; l < lanes; ++l) {
        const int rc = ensure_workspace(e, *e->more_lanes[l - 1], per);
        if (rc) return rc;
    }
    CK(cudaEventRecord(e->fork_ev, e->stream));
    int rc = AVA_OK;
    for (int l = 1; l < lanes; ++l)
        if (l * per < s->rows) CK(cudaStreamWaitEvent(e->more_lanes[l - 1]->lane_stream, e->fork_ev, 0));
    // the lanes are queued block by block in turn: queued one whole lane after the other, the second lane would start
    // only when the host has queued all of the first (a millisecond of a five-millisecond step)
    const int L = e->cfg.n_blocks;
    for (int b = 0; b < L && rc == AVA_OK; ++b)
        for (int l = 0; l < lanes && rc == AVA_OK; ++l) {
            const int r0 = l * per, n = std::min(per, s->rows - r0);
            if (n <= 0) break;
            Work& w = l == 0 ? static_cast<Work&>(*e) : *e->more_lanes[l - 1];
            rc = step_rows(e, w, l == 0 ? e->stream : w.lane_stream, s, r0, n, tok, logits, next, want_logits, T, all_logits, phase, b, b + 1 == L ? 1 << 30 : b + 1);
        }
    for (int l = 1; l < lanes; ++l) {
        if (l * per >= s->rows) break;
        Work& w = *e->more_lanes[l - 1];
        CK(cudaEventRecord(w.lane_done, w.lane_stream));
        CK(cudaStreamWaitEvent(e->stream, w.lane_done, 0));
    }
    e->cur = e->stream;
    e->cur_w = e;
    if (rc == AVA_OK && streams_state) {
        s->pend_set ^= 1;
        s->pending = true;
    }
    return rc;
}

// waits for the stream and turns the device status word into a return code (clearing it)
int finish(ava_engine* e) {
    CK(cudaMemcpyAsync(e->status_host, e->status.p, sizeof(uint32_t), cudaMemcpyDeviceToHost, e->stream));
    CK(cudaMemsetAsync(e->status.p, 0, sizeof(uint32_t), e->stream));
    CK(cudaStreamSynchronize(e->stream));
    const uint32_t st = *e->status_host;
    if (st & ST_WAIT_TIMEOUT) return e->fail(AVA_ERR_CUDA, "a bounded wait on a copy barrier ran out inside a kernel");
    if (st & ST_BAD_TOKEN) return e->fail(AVA_ERR_ARG, "a token id outside the vocabulary");
    if (st & ST_ENGRAM_FULL) return e->fail(AVA_ERR_CAPACITY, "the engram store had no room for a token");
    if (st & ST_NONFINITE) return e->fail(AVA_ERR_NONFINITE, "a gate, key or value of the fast-weight memory was not finite (the state has moved)");
    return AVA_OK;
}

int check_pair(ava_engine* e, ava_state* s) {
    if (!e) return AVA_ERR_ARG;
    if (!s || s->e != e) return e->fail(AVA_ERR_STATE, "the state belongs to another engine");
    if (!e->finalized) return e->fail(AVA_ERR_ARG, "engine not finalized");
    if (!e->blocker.empty()) return AVA_NOT_APPLICABLE;
    CK(cudaSetDevice(e->device));
    return ensure_workspace(e, *e, s->rows, s->rows);
}

struct StateSlice {
    Dev* buf = nullptr;
    size_t off = 0, count = 0;  // elements (floats, or store elements for the engram)
    bool eng = false;
    bool tiled = false;         // the fast weights: slice-major in device memory, natural [heads, hs, hs] outside
};

// where row `row`'s tensor `name` lives; for the engram the count is the tokens held times the row width
bool locate(const ava_state* s, int row, const std::string& name, StateSlice* out) {
    const ava_config& c = s->e->cfg;
    ava_state* ms = const_cast<ava_state*>(s);
    const size_t d = c.d, M = s->rows;
    if (name == "eng.k" || name == "eng.v") {
        if (c.eng_block < 0) return false;
        out->buf = name == "eng.k" ? &ms->eng_k : &ms->eng_v;
        out->eng = true;
        out->count = (size_t)s->n_host[row] * d;
        return true;
    }
    if (name == "v51.rh") {
        if (!c.rhythm) return false;
        out->buf = &ms->rh;
        out->off = (size_t)row * 2;
        out->count = 2;
        return true;
    }
    if (name.rfind("v51.", 0) == 0 && (c.dopamine || c.mood > 0)) {
        const std::string what = name.substr(4);
        const size_t k = what == "prev" ? d : what == "mood" ? (size_t)c.mood : 1;
        out->buf = what == "prev" ? &ms->sur_prev : what == "pvalid" ? &ms->sur_valid : what == "last_s" ? &ms->sur_last
                   : what == "mood" && c.mood > 0 ? &ms->mood : nullptr;
        out->off = (size_t)row * k;
        out->count = k;
        return out->buf != nullptr;
    }
    const size_t d1 = name.find('.'), d2 = name.rfind('.');
    if (d1 == std::string::npos || d2 == d1) return false;
    const std::string kind = name.substr(0, d1), what = name.substr(d2 + 1);
    const int i = std::atoi(name.substr(d1 + 1, d2 - d1 - 1).c_str());
    if (i < 0 || i >= c.n_blocks) return false;
    if (kind == "lif") {
        out->buf = what == "v" ? &ms->lif_v : what == "s" ? &ms->lif_s : what == "a" && c.alif ? &ms->lif_a : nullptr;
        out->off = ((size_t)i * M + row) * d;
        out->count = d;
        return out->buf != nullptr;
    }
    if (kind == "parts" && c.stp && (what == "stp_u" || what == "stp_x")) {
        out->buf = what == "stp_u" ? &ms->stp_u : &ms->stp_x;
        out->off = ((size_t)i * M + row) * d;
        out->count = d;
        return true;
    }
    if (kind == "mem" && c.fast_mem && (what == "f" || (what == "s" && c.mem_momentum > 0.0f))) {
        const size_t per = (size_t)d * c.head_size;  // nh * hs * hs
        out->buf = what == "f" ? &ms->mem_f : &ms->mem_s;
        out->off = ((size_t)i * M + row) * per;
        out->count = per;
        out->tiled = true;
        return true;
    }
    return false;
}

int alloc_state(ava_engine* e, int rows, int ring, int keep, ava_state** out) {
    const ava_config& c = e->cfg;
    std::unique_ptr<ava_state> s(new ava_state());
    s->e = e;
    s->rows = rows;
    s->ring = ring;
    s->keep = keep;
    const size_t M = rows, d = c.d, L = c.n_blocks, f = sizeof(float);
    CK(s->lif_v.alloc(L * M * d * f));
    CK(s->lif_s.alloc(L * M * d * f));
    if (c.alif) CK(s->lif_a.alloc(L * M * d * f));
    if (c.stp) {
        CK(s->stp_u.alloc(L * M * d * f));
        CK(s->stp_x.alloc(L * M * d * f));
    }
    if (c.rhythm) CK(s->rh.alloc(M * 2 * f));
    if (c.dopamine || c.mood > 0) {
        CK(s->sur_prev.alloc(M * d * f));
        CK(s->sur_valid.alloc(M * f));
        CK(s->sur_last.alloc(M * f));
        if (c.mood > 0) CK(s->mood.alloc(M * c.mood * f));
    }
    if (c.fast_mem) CK(s->mem_f.alloc(L * M * d * c.head_size * f));
    if (c.fast_mem && c.mem_momentum > 0.0f) CK(s->mem_s.alloc(L * M * d * c.head_size * f));
    if (c.fast_mem && !(c.mem_momentum > 0.0f)) CK(s->pend.alloc(2 * 5 * L * M * d * f));
    if (c.eng_block >= 0) {
        CK(s->eng_k.alloc(M * d * ring * s->kv_elem()));
        CK(s->eng_v.alloc(M * d * ring * s->kv_elem()));
        CK(s->eng_n.alloc(M * sizeof(int32_t)));
        CK(s->eng_start.alloc(M * sizeof(int32_t)));
    }
    s->n_host.assign(rows, 0);
    s->start_host.assign(rows, 0);
    s->seen.assign(rows, 0);
    *out = s.release();
    return AVA_OK;
}

int zero_state(ava_engine* e, ava_state* s) {
    for (Dev* b : {&s->lif_v, &s->lif_s, &s->lif_a, &s->mem_f, &s->mem_s, &s->stp_u, &s->sur_prev, &s->sur_valid, &s->sur_last, &s->mood, &s->rh, &s->eng_n,
                   &s->eng_start})
        if (b->p) CK(cudaMemsetAsync(b->p, 0, b->bytes, e->stream));
    if (s->stp_x.p) launch_fill(e->stream, s->stp_x.as<float>(), (int64_t)(s->stp_x.bytes / sizeof(float)), 1.0f);  // x starts at 1
    CK(cudaStreamSynchronize(e->stream));
    return AVA_OK;
}

// Applies the update the last decode step left pending to the fast weights, so that mem_f is the state every reader
// other than the next streaming pass expects (queued on the engine's stream; callers that read next synchronise anyway).
int flush_pending(ava_engine* e, ava_state* s) {
    if (!s->pending) return AVA_OK;
    const ava_config& c = e->cfg;
    CK(cudaSetDevice(e->device));
    for (int i = 0; i < c.n_blocks; ++i)
        launch_mem_flush(e->stream, s->mem_f.as<float>() + (size_t)i * s->rows * c.d * c.head_size, s->pend_at(s->pend_set, 0, i), s->pend_at(s->pend_set, 1, i),
                         s->pend_at(s->pend_set, 2, i), s->pend_at(s->pend_set, 3, i), s->pend_at(s->pend_set, 4, i), (int64_t)s->rows * e->nh(), c.head_size, e->cw);
    e->launches += c.n_blocks;
    s->pending = false;
    cudaError_t le = take_launch_error();
    if (le == cudaSuccess) le = cudaGetLastError();
    if (le != cudaSuccess) return e->cuda_fail(le, "kernel launch");
    return AVA_OK;
}

// copies row `src_row` of `src` into row `dst_row` of `dst` (same engine, same ring)
int copy_row(ava_engine* e, const ava_state* src, int src_row, ava_state* dst, int dst_row) {
    const ava_config& c = e->cfg;
    const size_t d = c.d, per = d * c.head_size, f = sizeof(float);
    for (int i = 0; i < c.n_blocks; ++i) {
        const size_t so = (size_t)i * src->rows + src_row, dn = (size_t)i * dst->rows + dst_row;
        CK(cudaMemcpyAsync(dst->lif_v.as<float>() + dn * d, src->lif_v.as<float>() + so * d, d * f, cudaMemcpyDeviceToDevice, e->stream));
        CK(cudaMemcpyAsync(dst->lif_s.as<float>() + dn * d, src->lif_s.as<float>() + so * d, d * f, cudaMemcpyDeviceToDevice, e->stream));
        if (c.alif)
            CK(cudaMemcpyAsync(dst->lif_a.as<float>() + dn * d, src->lif_a.as<float>() + so * d, d * f, cudaMemcpyDeviceToDevice, e->stream));
        if (c.stp) {
            CK(cudaMemcpyAsync(dst->stp_u.as<float>() + dn * d, src->stp_u.as<float>() + so * d, d * f, cudaMemcpyDeviceToDevice, e->stream));
            CK(cudaMemcpyAsync(dst->stp_x.as<float>() + dn * d, src->stp_x.as<float>() + so * d, d * f, cudaMemcpyDeviceToDevice, e->stream));
        }
        if (c.fast_mem)
            CK(cudaMemcpyAsync(dst->mem_f.as<float>() + dn * per, src->mem_f.as<float>() + so * per, per * f, cudaMemcpyDeviceToDevice, e->stream));
        if (c.fast_mem && c.mem_momentum > 0.0f)
            CK(cudaMemcpyAsync(dst->mem_s.as<float>() + dn * per, src->mem_s.as<float>() + so * per, per * f, cudaMemcpyDeviceToDevice, e->stream));
    }
    if (c.rhythm)
        CK(cudaMemcpyAsync(dst->rh.as<float>() + (size_t)dst_row * 2, src->rh.as<float>() + (size_t)src_row * 2, 2 * f, cudaMemcpyDeviceToDevice, e->stream));
    if (c.dopamine || c.mood > 0) {
        CK(cudaMemcpyAsync(dst->sur_prev.as<float>() + dst_row * d, src->sur_prev.as<float>() + src_row * d, d * f, cudaMemcpyDeviceToDevice, e->stream));
        CK(cudaMemcpyAsync(dst->sur_valid.as<float>() + dst_row, src->sur_valid.as<float>() + src_row, f, cudaMemcpyDeviceToDevice, e->stream));
        CK(cudaMemcpyAsync(dst->sur_last.as<float>() + dst_row, src->sur_last.as<float>() + src_row, f, cudaMemcpyDeviceToDevice, e->stream));
        if (c.mood > 0)
            CK(cudaMemcpyAsync(dst->mood.as<float>() + (size_t)dst_row * c.mood, src->mood.as<float>() + (size_t)src_row * c.mood, c.mood * f,
                               cudaMemcpyDeviceToDevice, e->stream));
    }
    if (c.eng_block >= 0) {
        const size_t rowb = d * src->ring * src->kv_elem();
        CK(cudaMemcpyAsync((char*)dst->eng_k.p + dst_row * rowb, (char*)src->eng_k.p + src_row * rowb, rowb, cudaMemcpyDeviceToDevice, e->stream));
        CK(cudaMemcpyAsync((char*)dst->eng_v.p + dst_row * rowb, (char*)src->eng_v.p + src_row * rowb, rowb, cudaMemcpyDeviceToDevice, e->stream));
        dst->n_host[dst_row] = src->n_host[src_row];
        dst->start_host[dst_row] = src->start_host[src_row];
    }
    dst->seen[dst_row] = src->seen[src_row];
    return AVA_OK;
}

int push_counts(ava_engine* e, ava_state* s) {
    if (e->cfg.eng_block < 0) return AVA_OK;
    CK(cudaMemcpyAsync(s->eng_n.p, s->n_host.data(), s->rows * sizeof(int32_t), cudaMemcpyHostToDevice, e->stream));
    CK(cudaMemcpyAsync(s->eng_start.p, s->start_host.data(), s->rows * sizeof(int32_t), cudaMemcpyHostToDevice, e->stream));
    CK(cudaStreamSynchronize(e->stream));
    return AVA_OK;
}

}  // namespace

// ================================================================================================ C ABI
extern "C" {

int ava_engine_create(const ava_config* cfg, int device, ava_engine** out) {
    if (!cfg || !out) return AVA_ERR_ARG;
    int count = 0;
    cudaError_t ce = cudaGetDeviceCount(&count);
    if (ce != cudaSuccess || count == 0) {
        g_create_error = std::string("no CUDA device: ") + cudaGetErrorString(ce) + " (this library has no CPU path)";
        return AVA_ERR_CUDA;
    }
    if (device < 0 || device >= count) {
        g_create_error = "device index out of range";
        return AVA_ERR_ARG;
    }
    std::unique_ptr<ava_engine> e(new ava_engine());
    e->cfg = *cfg;
    e->device = device;
    cudaSetDevice(device);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) e->sm_count = prop.multiProcessorCount;
    if ((ce = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking)) != cudaSuccess ||
        (ce = cudaMallocHost((void**)&e->status_host, sizeof(uint32_t))) != cudaSuccess || (ce = e->status.alloc(sizeof(uint32_t))) != cudaSuccess ||
        (ce = cudaMemset(e->status.p, 0, sizeof(uint32_t))) != cudaSuccess) {
        g_create_error = std::string("engine set-up: ") + cudaGetErrorString(ce);
        return AVA_ERR_CUDA;
    }
    e->cur = e->stream;
    e->cur_w = e.get();
    cudaStreamCreateWithFlags(&e->side_stream, cudaStreamNonBlocking);
    cudaEventCreateWithFlags(&e->side_go, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&e->side_done, cudaEventDisableTiming);
    const char* why = find_blocker(e->cfg, &e->cw, &e->rb);
    if (why) e->blocker = why;
    if (!why) {
        e->gate_cols = ((2 * e->nh() + 2 * cfg->gate_rank + 3) / 4) * 4;
        e->gate_chunk = 128;
        while (cfg->d % e->gate_chunk) e->gate_chunk /= 2;
        if (e->gate_cols > 224) e->blocker = "too many gate projection columns (heads and gate rank) for the gate kernel";
    }
    *out = e.release();
    return AVA_OK;
}

void ava_engine_destroy(ava_engine* e) {
    if (!e) return;
    cudaSetDevice(e->device);
    for (auto& w : e->more_lanes) {
        if (w->lane_stream) {
            cudaStreamSynchronize(w->lane_stream);
            cudaStreamDestroy(w->lane_stream);
        }
        if (w->lane_done) cudaEventDestroy(w->lane_done);
        if (w->side_stream) cudaStreamDestroy(w->side_stream);
        if (w->side_go) cudaEventDestroy(w->side_go);
        if (w->side_done) cudaEventDestroy(w->side_done);
    }
    if (e->side_stream) cudaStreamDestroy(e->side_stream);
    if (e->side_go) cudaEventDestroy(e->side_go);
    if (e->side_done) cudaEventDestroy(e->side_done);
    if (e->fork_ev) cudaEventDestroy(e->fork_ev);
    if (e->stream) {
        cudaStreamSynchronize(e->stream);
        cudaStreamDestroy(e->stream);
    }
    if (e->status_host) cudaFreeHost(e->status_host);
    delete e;
}

const char* ava_last_error(const ava_engine* e) { return e ? e->err.c_str() : g_create_error.c_str(); }
const char* ava_engine_blocker(const ava_engine* e) { return (e && !e->blocker.empty()) ? e->blocker.c_str() : nullptr; }

int ava_engine_set_f32(ava_engine* e, const char* name, const float* data, int64_t n) {
    if (!e || !name || !data) return AVA_ERR_ARG;
    const int64_t want = f32_len(e->cfg, name);
    if (want < 0) return e->fail(AVA_ERR_ARG, "unknown tensor %s", name);
    if (want != n) return e->fail(AVA_ERR_ARG, "%s: %lld values, want %lld", name, (long long)n, (long long)want);
    e->host_f32[name].assign(data, data + n);
    e->finalized = false;
    return AVA_OK;
}

int ava_engine_set_token_bytes(ava_engine* e, const uint8_t* bytes, const int64_t* offsets) {
    if (!e || !offsets) return AVA_ERR_ARG;
    const int V = e->cfg.vocab;
    for (int t = 0; t < V; ++t)
        if (offsets[t + 1] < offsets[t] || offsets[0] != 0) return e->fail(AVA_ERR_ARG, "token %d: offsets must start at 0 and not decrease", t);
    if (offsets[V] > 0 && !bytes) return AVA_ERR_ARG;
    e->tok_off.assign(offsets, offsets + V + 1);
    e->tok_bytes.assign(bytes, bytes + offsets[V]);
    e->finalized = false;
    return AVA_OK;
}

int ava_engine_set_q8(ava_engine* e, const char* name, const int8_t* q, const float* scale, int32_t din, int32_t dout) {
    if (!e || !name || !q || !scale) return AVA_ERR_ARG;
    int wi, wo;
    if (!q8_dims(e->cfg, name, &wi, &wo)) return e->fail(AVA_ERR_ARG, "unknown int8 matrix %s", name);
    if (wi != din || wo != dout) return e->fail(AVA_ERR_ARG, "%s: [%d, %d], want [%d, %d]", name, din, dout, wi, wo);
    HostQ& h = e->host_q8[name];
    h.din = din;
    h.dout = dout;
    h.q.assign(q, q + (size_t)din * dout);
    h.scale.assign(scale, scale + dout);
    e->finalized = false;
    return AVA_OK;
}

int ava_engine_set_q8_from_f32(ava_engine* e, const char* name, const float* w, int32_t din, int32_t dout) {
    if (!e || !name || !w || din <= 0 || dout <= 0) return AVA_ERR_ARG;
    std::vector<int8_t> q((size_t)din * dout);
    std::vector<float> sc(dout);
    quantize_int8(w, din, dout, q.data(), sc.data());
    return ava_engine_set_q8(e, name, q.data(), sc.data(), din, dout);
}

int ava_engine_finalize(ava_engine* e) {
    if (!e) return AVA_ERR_ARG;
    if (!e->blocker.empty()) {
        e->finalized = true;
        return AVA_NOT_APPLICABLE;
    }
    CK(cudaSetDevice(e->device));
    const ava_config& c = e->cfg;
    int rc;
    if ((rc = upload_f32(e, e->tok_emb, "tok_emb", true))) return rc;
    if ((rc = upload_f32(e, e->final_norm, "final.norm", true))) return rc;
    if (!e->host_q8.count("head")) {
        // the tied head: tok_emb^T quantised, one scale per vocabulary row (src/int8.rs:82-84)
        const std::vector<float>& emb = e->host_f32["tok_emb"];
        std::vector<float> et((size_t)c.d * c.vocab);
        for (int v = 0; v < c.vocab; ++v)
            for (int j = 0; j < c.d; ++j) et[(size_t)j * c.vocab + v] = emb[(size_t)v * c.d + j];
        if ((rc = ava_engine_set_q8_from_f32(e, "head", et.data(), c.d, c.vocab))) return rc;
    }
    if ((rc = upload_q8(e, e->head, {"head"}))) return rc;
    e->blocks.clear();
    for (int i = 0; i < c.n_blocks; ++i) {
        e->blocks.emplace_back(new BlockDev());
        BlockDev& b = *e->blocks.back();
        const std::string p = "b" + std::to_string(i) + ".";
        if ((rc = upload_f32(e, b.mem_norm, p + "mem.norm", true))) return rc;
        {
            // leak and adaptation rate are sigmoids of their parameters (src/model/fstep/arch.rs:640,660)
            auto it = e->host_f32.find(p + "mem.beta");
            if (it == e->host_f32.end()) return e->fail(AVA_ERR_MISSING, "missing tensor %smem.beta", p.c_str());
            std::vector<float> beta(it->second.size());
            for (size_t k = 0; k < beta.size(); ++k) beta[k] = ava::sigmoid(it->second[k]);
            if ((rc = upload(e, b.beta, beta.data(), beta.size() * sizeof(float)))) return rc;
            if (c.alif) {
                auto ir = e->host_f32.find(p + "mem.arho");
                if (ir == e->host_f32.end()) return e->fail(AVA_ERR_MISSING, "missing tensor %smem.arho", p.c_str());
                std::vector<float> rho(ir->second.size());
                for (size_t k = 0; k < rho.size(); ++k) rho[k] = ava::sigmoid(ir->second[k]);
                if ((rc = upload(e, b.rho, rho.data(), rho.size() * sizeof(float)))) return rc;
                if ((rc = upload_f32(e, b.again, p + "mem.again", true))) return rc;
            }
        }
        if ((rc = upload_f32(e, b.theta, p + "mem.theta", c.theta != 0))) return rc;
        if (c.dendrite && c.fast_mem) {
            if ((rc = upload_f32(e, b.dend_a, p + "v51.dend_a", true))) return rc;
            if ((rc = upload_f32(e, b.dend_b, p + "v51.dend_b", true))) return rc;
        }
        if (c.dopamine && i > 0) {
            if ((rc = upload_f32(e, b.da_w, p + "v51.da_w", true))) return rc;
            if ((rc = upload_f32(e, b.da_c, p + "v51.da_c", true))) return rc;
        }
        if (c.mood > 0 && i > 0 && (rc = upload_f32(e, b.mood_g, p + "v51.mood_g", true))) return rc;
        if (c.rhythm) {
            if ((rc = upload_f32(e, b.rh_w, p + "v51.rh_w", true))) return rc;
            if ((rc = upload_f32(e, b.rh_r, p + "v51.rh_r", true))) return rc;
        }
        if (c.stp) {
            // U, F, D are sigmoids of their parameters (src/model/fstep/arch_f3.rs:82)
            struct P { Dev* d; const char* n; bool sig; };
            for (const P& q : {P{&b.stp_U, "parts.stp.u_param", true}, P{&b.stp_F, "parts.stp.f_param", true}, P{&b.stp_D, "parts.stp.d_param", true},
                               P{&b.stp_mix, "parts.stp.mix", false}}) {
                auto it = e->host_f32.find(p + q.n);
                if (it == e->host_f32.end()) return e->fail(AVA_ERR_MISSING, "missing tensor %s%s", p.c_str(), q.n);
                std::vector<float> v(it->second);
                if (q.sig)
                    for (float& t : v) t = ava::sigmoid(t);
                if ((rc = upload(e, *q.d, v.data(), v.size() * sizeof(float)))) return rc;
            }
        }
        if ((rc = upload_f32(e, b.mlp_norm, p + "mlp.norm", true))) return rc;
        if (c.fast_mem) {
        if ((rc = upload_f32(e, b.hebb_norm, p + "hebb.norm", true))) return rc;
        struct F { Dev* d; const char* n; };
        for (const F& f : {F{&b.ba, "hebb.ba"}, F{&b.bb, "hebb.bb"}, F{&b.wa2, "hebb.wa2"}, F{&b.wb2, "hebb.wb2"}, F{&b.off, "hebb.off"}})
            if ((rc = upload_f32(e, *f.d, p + f.n, true))) return rc;
        {
            // the gates' first-stage projections side by side [d][wa1 | wb1 | wa | wb | zero padding]: one staged stream
            // (the low-rank parts first, so that each row's z1 values start on a 16-byte boundary)
            const int nh = e->nh(), rk = c.gate_rank, ncp = e->gate_cols;
            std::vector<float> gw((size_t)c.d * ncp, 0.0f);
            struct G { const char* n; int w; };
            int c0 = 0;
            for (const G& gpart : {G{"hebb.wa1", rk}, G{"hebb.wb1", rk}, G{"hebb.wa", nh}, G{"hebb.wb", nh}}) {
                auto it = e->host_f32.find(p + gpart.n);
                if (it == e->host_f32.end()) return e->fail(AVA_ERR_MISSING, "missing tensor %s%s", p.c_str(), gpart.n);
                for (int j = 0; j < c.d; ++j)
                    for (int k = 0; k < gpart.w; ++k) gw[(size_t)j * ncp + c0 + k] = it->second[(size_t)j * gpart.w + k];
                c0 += gpart.w;
            }
            if ((rc = upload(e, b.gate_w, gw.data(), gw.size() * sizeof(float)))) return rc;
        }
        if ((rc = upload_f32(e, b.vres, p + "hebb.vres", c.value_residual && i > 0))) return rc;
        std::vector<std::string> pj = {p + "hebb.wq", p + "hebb.wk", p + "hebb.wv", p + "hebb.we"};
        if (c.out_gate) pj.push_back(p + "hebb.wg");
        if ((rc = upload_q8(e, b.proj, pj))) return rc;
        if ((rc = upload_q8(e, b.wo, {p + "hebb.wo"}))) return rc;
        }
        if ((rc = upload_f32(e, b.dense, p + "dense", c.dense != 0))) return rc;
        if ((rc = upload_q8(e, b.win, {p + "mem.win"}))) return rc;
        if ((rc = upload_q8(e, b.wout, {p + "mem.wout"}))) return rc;
        if (i == c.eng_block) {
            if ((rc = upload_f32(e, b.eng_norm, p + "eng.norm", true))) return rc;
            if ((rc = upload_q8(e, b.eqkv, {p + "eng.wq", p + "eng.wk", p + "eng.wv"}))) return rc;
            if ((rc = upload_q8(e, b.ewo, {p + "eng.wo"}))) return rc;
        }
        if ((rc = upload_q8(e, b.w1, {p + "mlp.w1"}))) return rc;
        if ((rc = upload_q8(e, b.w2, {p + "mlp.w2"}))) return rc;
    }
    if (c.neuromod > 0) {
        if ((rc = upload_f32(e, e->nm_norm, "nm.norm", true))) return rc;
        if ((rc = upload_f32(e, e->nm_bn, "nm.bn", true))) return rc;
        auto it = e->host_f32.find("nm.wn");
        if (it == e->host_f32.end()) return e->fail(AVA_ERR_MISSING, "missing tensor nm.wn");
        std::vector<float> w4((size_t)c.d * 4, 0.0f);  // [d][k] with the columns padded to four
        for (int j = 0; j < c.d; ++j)
            for (int k = 0; k < c.neuromod; ++k) w4[(size_t)j * 4 + k] = it->second[(size_t)j * c.neuromod + k];
        if ((rc = upload(e, e->nm_wn, w4.data(), w4.size() * sizeof(float)))) return rc;
    }
    if (c.rhythm) {
        if ((rc = upload_f32(e, e->rhy_lw, "v51.rhythm.lw", true))) return rc;
        if ((rc = upload_f32(e, e->rhy_br, "v51.rhythm.br", true))) return rc;
        auto it = e->host_f32.find("v51.rhythm.wr");
        if (it == e->host_f32.end()) return e->fail(AVA_ERR_MISSING, "missing tensor v51.rhythm.wr");
        std::vector<float> w4((size_t)c.d * 4, 0.0f);  // [d][2] with the columns padded to four
        for (int j = 0; j < c.d; ++j)
            for (int k = 0; k < 2; ++k) w4[(size_t)j * 4 + k] = it->second[(size_t)j * 2 + k];
        if ((rc = upload(e, e->rhy_wr, w4.data(), w4.size() * sizeof(float)))) return rc;
    }
    if (c.mood > 0) {
        if ((rc = upload_f32(e, e->mood_lam, "v51.mood.lam", true))) return rc;
        if ((rc = upload_f32(e, e->mood_win, "v51.mood.win", true))) return rc;
        if ((rc = upload_f32(e, e->mood_bin, "v51.mood.bin", true))) return rc;
    }
    if (c.thalamus) {
        if ((rc = upload_f32(e, e->th_read, "th.read", true))) return rc;
        if ((rc = upload_f32(e, e->th_gate, "th.gate", true))) return rc;
        if ((rc = upload_f32(e, e->th_bias, "th.bias", true))) return rc;
    }
    if (c.letters) {
        // R (src/model/fstep/arch_f2.rs:34-60, src/v51.rs:449-469): a token's share of its input depends on the token alone,
        // so the whole table is built here, once, with the arithmetic the kernels share with the host: per token
        // l = (0 + m_0 tanh((E[b_0] + Q[e_0]) + P[0]) + ... over 16 places) * inv, b the bytes of its spelling, e their
        // places counted from the end, m = 1 for a place in use, inv = 1 / sqrt(places in use); then l Wo in the one-row
        // order (Wo[0] l_0, then one fused multiply-add per further input)
        if (e->tok_off.size() != (size_t)c.vocab + 1) return e->fail(AVA_ERR_MISSING, "--letters: the tokens' spellings are not set (ava_engine_set_token_bytes)");
        const char* names[4] = {"v51.letters.byte", "v51.letters.pos", "v51.letters.end", "v51.letters.wo"};
        const std::vector<float>* w[4];
        for (int q = 0; q < 4; ++q) {
            auto it = e->host_f32.find(names[q]);
            if (it == e->host_f32.end()) return e->fail(AVA_ERR_MISSING, "missing tensor %s", names[q]);
            w[q] = &it->second;
        }
        const float *E = w[0]->data(), *P = w[1]->data(), *Q = w[2]->data(), *Wo = w[3]->data();
        constexpr int DL = 64, LM = 16;
        const int d = c.d;
        std::vector<float> table((size_t)c.vocab * d);
        for (int t = 0; t < c.vocab; ++t) {
            const int64_t len = e->tok_off[t + 1] - e->tok_off[t];
            const int used = (int)std::min<int64_t>(len, LM);
            const float inv = used > 0 ? ava::div(1.0f, ava::root((float)used)) : 0.0f;
            float l[DL];
            for (int cc = 0; cc < DL; ++cc) l[cc] = 0.0f;
            for (int j = 0; j < LM; ++j) {
                const int b = j < used ? e->tok_bytes[e->tok_off[t] + j] : 0;
                const int k = j < used ? (int)std::min<int64_t>(len - 1 - j, LM - 1) : 0;
                const float m = j < used ? 1.0f : 0.0f;
                for (int cc = 0; cc < DL; ++cc) {
                    const float sv = ava::tanhf_(ava::add(ava::add(E[b * DL + cc], Q[k * DL + cc]), P[j * DL + cc]));
                    l[cc] = ava::add(l[cc], ava::mul(sv, m));
                }
            }
            for (int cc = 0; cc < DL; ++cc) l[cc] = ava::mul(l[cc], inv);
            float* out = &table[(size_t)t * d];
            for (int cc = 0; cc < d; ++cc) out[cc] = ava::mul(Wo[cc], l[0]);
            for (int j = 1; j < DL; ++j)
                for (int cc = 0; cc < d; ++cc) out[cc] = ava::fma(Wo[(size_t)j * d + cc], l[j], out[cc]);
        }
        if ((rc = upload(e, e->letters, table.data(), table.size() * sizeof(float)))) return rc;
    }
    if (c.cb_units > 0) {
        if ((rc = upload_f32(e, e->cb_w, "cbh.wo", true))) return rc;
        // the fixed wiring (src/v51b.rs:241-266, seed and fan-in :47-49): Marsaglia's xorshift64 (13, 7, 17) from seed | 1;
        // per unit four distinct inputs of the 2 d (a draw modulo 2 d, redrawn while already picked), then per input one more
        // draw whose lowest bit gives the sign of 1/2
        const int G = c.cb_units, inputs = 2 * c.d, fan = 4;
        std::vector<uint32_t> idx;
        std::vector<float> sg;
        uint64_t sd = 0x51B0CE7Eull | 1;
        auto next = [&]() {
            sd ^= sd << 13;
            sd ^= sd >> 7;
            sd ^= sd << 17;
            return sd;
        };
        const float amp = 1.0f / std::sqrt((float)fan);
        for (int u = 0; u < G; ++u) {
            uint32_t picked[4];
            int np = 0;
            while (np < std::min(fan, inputs)) {
                const uint32_t r = (uint32_t)(next() % (uint64_t)inputs);
                bool seen = false;
                for (int q = 0; q < np; ++q) seen |= picked[q] == r;
                if (!seen) picked[np++] = r;
            }
            for (int q = 0; q < np; ++q) {
                idx.push_back(picked[q]);
                sg.push_back((next() & 1) == 0 ? amp : -amp);
            }
        }
        if ((rc = upload(e, e->cb_idx, idx.data(), idx.size() * sizeof(uint32_t)))) return rc;
        if ((rc = upload(e, e->cb_sgn, sg.data(), sg.size() * sizeof(float)))) return rc;
    }
    if ((c.dendrite && c.fast_mem) || c.thalamus || c.cb_units > 0 || c.rhythm) {
        const std::vector<float> one((size_t)c.d, 1.0f);
        if ((rc = upload(e, e->ones, one.data(), one.size() * sizeof(float)))) return rc;
    }
    {
        // what `Model::fingerprint` hashes (src/state.rs:1075-1091): the configuration, every 97th value of tok_emb, final.norm,
        // every 101st value of each block's w2, FNV-1a over their bytes.  The reference hashes the Debug text of its Config
        // and the f32 w2; here the configuration's fields and the int8 w2 with its scales, so the two values differ: a state
        // file is tied to the engine's model, not exchangeable with the reference's check (see ava_state_save).
        uint64_t h = 0xcbf29ce484222325ull;
        auto bytes = [&](const void* p, size_t n) {
            const unsigned char* b = static_cast<const unsigned char*>(p);
            for (size_t k = 0; k < n; ++k) h = (h ^ b[k]) * 0x100000001b3ull;
        };
        bytes(&e->cfg, sizeof(ava_config));
        const auto& te = e->host_f32["tok_emb"];
        for (size_t k = 0; k < te.size(); k += 97) bytes(&te[k], 4);
        const auto& fn = e->host_f32["final.norm"];
        for (size_t k = 0; k < fn.size(); ++k) bytes(&fn[k], 4);
        for (int i = 0; i < c.n_blocks; ++i) {
            const HostQ& w2 = e->host_q8["b" + std::to_string(i) + ".mlp.w2"];
            for (size_t k = 0; k < w2.q.size(); k += 101) bytes(&w2.q[k], 1);
            bytes(w2.scale.data(), w2.scale.size() * 4);
        }
        e->fingerprint = h;
    }
    // the host copies are no longer needed
    e->host_f32.clear();
    e->host_q8.clear();
    e->finalized = true;
    return AVA_OK;
}

int ava_state_new(ava_engine* e, int32_t rows, int32_t max_ctx, ava_state** out) {
    if (!e || !out || rows <= 0) return AVA_ERR_ARG;
    if (!e->finalized) return e->fail(AVA_ERR_ARG, "engine not finalized");
    if (!e->blocker.empty()) return AVA_NOT_APPLICABLE;
    CK(cudaSetDevice(e->device));
    const ava_config& c = e->cfg;
    // a capped store reads cap + 1 tokens before it drops the oldest (src/model/fstep/arch.rs:962-964)
    const int ring = c.eng_block < 0 ? 0 : (c.eng_cap > 0 ? c.eng_cap + 1 : std::max(1, max_ctx));
    const int keep = c.eng_cap > 0 ? c.eng_cap : ring;
    ava_state* s = nullptr;
    int rc = alloc_state(e, rows, ring, keep, &s);
    if (rc) return rc;
    if ((rc = zero_state(e, s))) {
        delete s;
        return rc;
    }
    *out = s;
    return AVA_OK;
}

void ava_state_destroy(ava_state* s) {
    if (!s) return;
    cudaSetDevice(s->e->device);
    cudaStreamSynchronize(s->e->stream);
    delete s;
}

int32_t ava_state_rows(const ava_state* s) { return s ? s->rows : 0; }

int ava_state_select(const ava_state* s, const int32_t* idx, int32_t n, ava_state** out) {
    if (!s || !idx || !out || n <= 0) return AVA_ERR_ARG;
    ava_engine* e = s->e;
    for (int i = 0; i < n; ++i)
        if (idx[i] < 0 || idx[i] >= s->rows) return e->fail(AVA_ERR_ARG, "select: row %d of %d", idx[i], s->rows);
    CK(cudaSetDevice(e->device));
    ava_state* o = nullptr;
    int rc = flush_pending(e, const_cast<ava_state*>(s));  // the copy takes the fast weights as they are in memory
    if (rc) return rc;
    if ((rc = alloc_state(e, n, s->ring, s->keep, &o))) return rc;
    for (int i = 0; i < n && !rc; ++i) rc = copy_row(e, s, idx[i], o, i);
    if (!rc) rc = push_counts(e, o);
    if (rc) {
        delete o;
        return rc;
    }
    *out = o;
    return AVA_OK;
}

int ava_state_cat(const ava_state* const* parts, int32_t n, ava_state** out) {
    if (!parts || n <= 0 || !out || !parts[0]) return AVA_ERR_ARG;
    ava_engine* e = parts[0]->e;
    int rows = 0;
    for (int i = 0; i < n; ++i) {
        if (!parts[i] || parts[i]->e != e) return e->fail(AVA_ERR_STATE, "cat: states of different engines");
        if (parts[i]->ring != parts[0]->ring) return e->fail(AVA_ERR_STATE, "cat: states with different engram capacities");
        rows += parts[i]->rows;
    }
    CK(cudaSetDevice(e->device));
    ava_state* o = nullptr;
    int rc = AVA_OK;
    for (int i = 0; i < n && !rc; ++i) rc = flush_pending(e, const_cast<ava_state*>(parts[i]));
    if (rc) return rc;
    if ((rc = alloc_state(e, rows, parts[0]->ring, parts[0]->keep, &o))) return rc;
    int at = 0;
    for (int i = 0; i < n && !rc; ++i)
        for (int r = 0; r < parts[i]->rows && !rc; ++r) rc = copy_row(e, parts[i], r, o, at++);
    if (!rc) rc = push_counts(e, o);
    if (rc) {
        delete o;
        return rc;
    }
    *out = o;
    return AVA_OK;
}

uint64_t ava_engine_fingerprint(const ava_engine* e) { return e ? e->fingerprint : 0; }
ava_engine* ava_state_engine(const ava_state* s) { return s ? s->e : nullptr; }
int ava_state_set_seen(ava_state* s, int32_t row, int64_t seen) {
    if (!s || row < 0 || row >= s->rows || seen < 0) return AVA_ERR_ARG;
    s->seen[row] = seen;
    return AVA_OK;
}

int64_t ava_state_seen(const ava_state* s, int32_t row) { return (s && row >= 0 && row < s->rows) ? s->seen[row] : -1; }

int64_t ava_state_len(const ava_state* s, int32_t row, const char* name) {
    StateSlice sl;
    if (!s || !name || row < 0 || row >= s->rows || !locate(s, row, name, &sl)) return -1;
    return (int64_t)sl.count;
}

int ava_state_export(const ava_state* s, int32_t row, const char* name, float* out) {
    if (!s || !name || !out) return AVA_ERR_ARG;
    ava_engine* e = s->e;
    StateSlice sl;
    if (row < 0 || row >= s->rows || !locate(s, row, name, &sl)) return e->fail(AVA_ERR_ARG, "no state tensor %s of row %d", name, row);
    CK(cudaSetDevice(e->device));
    if (sl.tiled) {
        const int frc = flush_pending(e, const_cast<ava_state*>(s));
        if (frc) return frc;
    }
    CK(cudaStreamSynchronize(e->stream));
    if (sl.tiled) {
        Dev tmp;
        CK(tmp.alloc(sl.count * sizeof(float)));
        launch_retile(e->stream, sl.buf->as<float>() + sl.off, tmp.as<float>(), e->nh(), e->cfg.head_size, e->cw, 0);
        CK(cudaStreamSynchronize(e->stream));
        CK(cudaMemcpy(out, tmp.p, sl.count * sizeof(float), cudaMemcpyDeviceToHost));
        return AVA_OK;
    }
    if (!sl.eng) {
        CK(cudaMemcpy(out, sl.buf->as<float>() + sl.off, sl.count * sizeof(float), cudaMemcpyDeviceToHost));
        return AVA_OK;
    }
    // the ring [heads, ring, hs] unrolled oldest first into [heads, n, hs], widened to f32
    const ava_config& c = e->cfg;
    const int ehs = c.eng_head_size, enh = c.d / ehs, n = s->n_host[row], ring = s->ring, start = s->start_host[row];
    const size_t rowe = (size_t)c.d * ring;
    std::vector<unsigned char> raw(rowe * s->kv_elem());
    CK(cudaMemcpy(raw.data(), (char*)sl.buf->p + row * rowe * s->kv_elem(), raw.size(), cudaMemcpyDeviceToHost));
    for (int hh = 0; hh < enh; ++hh)
        for (int j = 0; j < n; ++j)
            for (int x = 0; x < ehs; ++x) {
                const size_t src = ((size_t)hh * ring + (start + j) % ring) * ehs + x;
                out[((size_t)hh * n + j) * ehs + x] = c.eng_store_bf16 ? ava::bf16_to_f(reinterpret_cast<uint16_t*>(raw.data())[src])
                                                                      : reinterpret_cast<float*>(raw.data())[src];
            }
    return AVA_OK;
}

int ava_state_import(ava_state* s, int32_t row, const char* name, const float* in, int64_t n) {
    if (!s || !name || !in) return AVA_ERR_ARG;
    ava_engine* e = s->e;
    StateSlice sl;
    if (row < 0 || row >= s->rows || !locate(s, row, name, &sl)) return e->fail(AVA_ERR_ARG, "no state tensor %s of row %d", name, row);
    CK(cudaSetDevice(e->device));
    if (sl.tiled) {
        const int frc = flush_pending(e, s);  // the other rows' pending updates must not be lost, nor applied to what is written now
        if (frc) return frc;
    }
    CK(cudaStreamSynchronize(e->stream));
    if (!sl.eng) {
        if ((int64_t)sl.count != n) return e->fail(AVA_ERR_ARG, "%s: %lld values, want %lld", name, (long long)n, (long long)sl.count);
        if (sl.tiled) {
            Dev tmp;
            CK(tmp.alloc(sl.count * sizeof(float)));
            CK(cudaMemcpy(tmp.p, in, n * sizeof(float), cudaMemcpyHostToDevice));
            launch_retile(e->stream, tmp.as<float>(), sl.buf->as<float>() + sl.off, e->nh(), e->cfg.head_size, e->cw, 1);
            CK(cudaStreamSynchronize(e->stream));
            return AVA_OK;
        }
        CK(cudaMemcpy(sl.buf->as<float>() + sl.off, in, n * sizeof(float), cudaMemcpyHostToDevice));
        return AVA_OK;
    }
    const ava_config& c = e->cfg;
    const int ehs = c.eng_head_size, enh = c.d / ehs, ring = s->ring;
    if (n % c.d) return e->fail(AVA_ERR_ARG, "%s: not whole tokens", name);
    const int tokens = (int)(n / c.d);
    if (tokens > s->keep) return e->fail(AVA_ERR_CAPACITY, "%s: %d tokens, room for %d", name, tokens, s->keep);
    const size_t rowe = (size_t)c.d * ring;
    std::vector<unsigned char> raw(rowe * s->kv_elem(), 0);
    for (int hh = 0; hh < enh; ++hh)
        for (int j = 0; j < tokens; ++j)
            for (int x = 0; x < ehs; ++x) {
                const float v = in[((size_t)hh * tokens + j) * ehs + x];
                const size_t dst = ((size_t)hh * ring + j) * ehs + x;
                if (c.eng_store_bf16)
                    reinterpret_cast<uint16_t*>(raw.data())[dst] = ava::f_to_bf16(v);
                else
                    reinterpret_cast<float*>(raw.data())[dst] = v;
            }
    CK(cudaMemcpy((char*)sl.buf->p + row * rowe * s->kv_elem(), raw.data(), raw.size(), cudaMemcpyHostToDevice));
    // keys and values are imported one after the other: the count follows whichever came last
    s->n_host[row] = tokens;
    s->start_host[row] = 0;
    return push_counts(e, s);
}

int ava_step_device(ava_engine* e, ava_state* s, const uint32_t* tok_device, float* logits_device, uint32_t* next_device) {
    int rc = check_pair(e, s);
    if (rc) return rc;
    if (!tok_device) return e->fail(AVA_ERR_ARG, "no tokens");
    return step_device(e, s, tok_device, logits_device, next_device, logits_device != nullptr);
}

int ava_sync(ava_engine* e) {
    if (!e) return AVA_ERR_ARG;
    CK(cudaSetDevice(e->device));
    return finish(e);
}

// ---- commit at the end (src/model/fstep/arch.rs:1059-1069: "everything computed: the State moves on") ----------------
// The kernels update the carried state as they go.  For a state with commit_at_end set, a host-facing call brackets its
// work: the small carried tensors (membranes, traces, the parts' states, the engram's counts) are copied aside first;
// the fast weights, the bulk of the state, are not copied for a one-token step: the streaming pass reads one copy and
// writes the other, and the two change places only when the call has succeeded (no extra traffic, twice the memory).
// A prompt (several tokens per row) or a memory with momentum works in place, so the fast weights are copied aside
// whole for such a call.  The engram's keys and values need no copy: a token only ever fills a free slot, and the
// counts say which slots hold tokens.  When the call fails after work was queued (a non-finite gate, a full store, a
// wait that ran out), everything is put back and the state is as it was before the call.
struct Txn {
    bool active = false, pingpong = false, whole = false, was_pending = false;
    int pend_set = 0;
    int64_t shard_pos = 0;
    std::vector<int32_t> n_host, start_host;
    std::vector<int64_t> seen;
    Dev whole_f, whole_s, whole_pend;
};

std::vector<Dev*> small_carried(ava_state* s) {
    return {&s->lif_v, &s->lif_s, &s->lif_a, &s->stp_u, &s->stp_x, &s->rh, &s->sur_prev, &s->sur_valid, &s->sur_last, &s->mood, &s->eng_n, &s->eng_start};
}

int txn_begin(ava_engine* e, ava_state* s, bool one_token, Txn& t) {
    if (!s->commit_at_end) return AVA_OK;
    const ava_config& c = e->cfg;
    t.active = true;
    t.was_pending = s->pending;
    t.pend_set = s->pend_set;
    t.shard_pos = s->shard_pos;
    t.n_host = s->n_host; t.start_host = s->start_host; t.seen = s->seen;
    size_t need = 0;
    for (Dev* d : small_carried(s)) need += (d->bytes + 255) & ~(size_t)255;
    if (s->snap.bytes < need) CK(s->snap.alloc(need));
    size_t at = 0;
    for (Dev* d : small_carried(s)) {
        if (d->bytes) CK(cudaMemcpyAsync((char*)s->snap.p + at, d->p, d->bytes, cudaMemcpyDeviceToDevice, e->stream));
        at += (d->bytes + 255) & ~(size_t)255;
    }
    t.pingpong = one_token && c.fast_mem && !(c.mem_momentum > 0.0f);
    if (t.pingpong) {
        if (!s->mem_f_alt.p) CK(s->mem_f_alt.alloc(s->mem_f.bytes));
        s->txn_pingpong = true;
    } else if (c.fast_mem) {
        t.whole = true;
        CK(t.whole_f.alloc(s->mem_f.bytes));
        CK(cudaMemcpyAsync(t.whole_f.p, s->mem_f.p, s->mem_f.bytes, cudaMemcpyDeviceToDevice, e->stream));
        if (s->mem_s.bytes) {
            CK(t.whole_s.alloc(s->mem_s.bytes));
            CK(cudaMemcpyAsync(t.whole_s.p, s->mem_s.p, s->mem_s.bytes, cudaMemcpyDeviceToDevice, e->stream));
        }
        if (s->pend.bytes) {
            CK(t.whole_pend.alloc(s->pend.bytes));
            CK(cudaMemcpyAsync(t.whole_pend.p, s->pend.p, s->pend.bytes, cudaMemcpyDeviceToDevice, e->stream));
        }
    }
    return AVA_OK;
}

// rc: what the call is about to return.  Success: the second copy of the fast weights becomes the state's.  Failure:
// everything goes back (the stream is idle by then: finish() has waited, or nothing was queued after an early refusal).
int txn_end(ava_engine* e, ava_state* s, Txn& t, int rc) {
    if (!t.active) return rc;
    s->txn_pingpong = false;
    if (rc == AVA_OK) {
        if (t.pingpong && t.was_pending) {   // the pass wrote the new weights there
            std::swap(s->mem_f.p, s->mem_f_alt.p);
            std::swap(s->mem_f.bytes, s->mem_f_alt.bytes);
        }
        return rc;
    }
    cudaStreamSynchronize(e->stream);
    size_t at = 0;
    for (Dev* d : small_carried(s)) {
        if (d->bytes) cudaMemcpyAsync(d->p, (char*)s->snap.p + at, d->bytes, cudaMemcpyDeviceToDevice, e->stream);
        at += (d->bytes + 255) & ~(size_t)255;
    }
    if (t.whole) {
        cudaMemcpyAsync(s->mem_f.p, t.whole_f.p, s->mem_f.bytes, cudaMemcpyDeviceToDevice, e->stream);
        if (s->mem_s.bytes) cudaMemcpyAsync(s->mem_s.p, t.whole_s.p, s->mem_s.bytes, cudaMemcpyDeviceToDevice, e->stream);
        if (s->pend.bytes) cudaMemcpyAsync(s->pend.p, t.whole_pend.p, s->pend.bytes, cudaMemcpyDeviceToDevice, e->stream);
    }
    cudaStreamSynchronize(e->stream);
    s->pending = t.was_pending;
    s->pend_set = t.pend_set;
    s->shard_pos = t.shard_pos;
    s->n_host = t.n_host; s->start_host = t.start_host; s->seen = t.seen;
    return rc;
}

int ava_state_set_commit_at_end(ava_state* s, int32_t on) {
    if (!s) return AVA_ERR_ARG;
    s->commit_at_end = on != 0;
    if (!on) {
        s->mem_f_alt.release();
        s->snap.release();
    }
    return AVA_OK;
}

int ava_step(ava_engine* e, ava_state* s, const uint32_t* tok, float* logits) {
    int rc = check_pair(e, s);
    if (rc) return rc;
    if (!tok || !logits) return e->fail(AVA_ERR_ARG, "null buffer");
    for (int r = 0; r < s->rows; ++r)
        if (tok[r] >= (uint32_t)e->cfg.vocab) return e->fail(AVA_ERR_ARG, "token %u of row %d outside the vocabulary", tok[r], r);
    Txn txn;
    if ((rc = txn_begin(e, s, true, txn))) return rc;
    auto body = [&]() -> int {
        CK(cudaMemcpyAsync(e->tok.p, tok, s->rows * sizeof(uint32_t), cudaMemcpyHostToDevice, e->stream));
        if (const int rs = step_device(e, s, e->tok.as<uint32_t>(), e->logits.as<float>(), nullptr, true)) return rs;
        CK(cudaMemcpyAsync(logits, e->logits.p, (size_t)s->rows * e->cfg.vocab * sizeof(float), cudaMemcpyDeviceToHost, e->stream));
        return finish(e);
    };
    return txn_end(e, s, txn, body());
}

int ava_step_greedy(ava_engine* e, ava_state* s, const uint32_t* tok, uint32_t* next) {
    int rc = check_pair(e, s);
    if (rc) return rc;
    if (!tok || !next) return e->fail(AVA_ERR_ARG, "null buffer");
    for (int r = 0; r < s->rows; ++r)
        if (tok[r] >= (uint32_t)e->cfg.vocab) return e->fail(AVA_ERR_ARG, "token %u of row %d outside the vocabulary", tok[r], r);
    Txn txn;
    if ((rc = txn_begin(e, s, true, txn))) return rc;
    auto body = [&]() -> int {
        CK(cudaMemcpyAsync(e->tok.p, tok, s->rows * sizeof(uint32_t), cudaMemcpyHostToDevice, e->stream));
        if (const int rs = step_device(e, s, e->tok.as<uint32_t>(), nullptr, e->next.as<uint32_t>(), false)) return rs;
        CK(cudaMemcpyAsync(next, e->next.p, s->rows * sizeof(uint32_t), cudaMemcpyDeviceToHost, e->stream));
        return finish(e);
    };
    return txn_end(e, s, txn, body());
}

int ava_step_sample(ava_engine* e, ava_state* s, const uint32_t* tok, float temperature, int32_t top_k, const double* uniform, uint32_t* next) {
    if (!(temperature > 0.0f)) return ava_step_greedy(e, s, tok, next);
    int rc = check_pair(e, s);
    if (rc) return rc;
    if (!tok || !next || !uniform) return e->fail(AVA_ERR_ARG, "null buffer");
    for (int r = 0; r < s->rows; ++r)
        if (tok[r] >= (uint32_t)e->cfg.vocab) return e->fail(AVA_ERR_ARG, "token %u of row %d outside the vocabulary", tok[r], r);
    // asked before anything moves: a refusal leaves the state as it was
    if (!sample_covered(e->cfg.vocab, top_k))
        return e->fail(AVA_NOT_APPLICABLE, "the device sampler does not cover this vocabulary or top_k (top_k above 1024, or a vocabulary beyond its shared memory): pick on the host (ava_step + ava_pick)");
    Txn txn;
    if ((rc = txn_begin(e, s, true, txn))) return rc;
    auto body = [&]() -> int {
        CK(cudaMemcpyAsync(e->tok.p, tok, s->rows * sizeof(uint32_t), cudaMemcpyHostToDevice, e->stream));
        CK(cudaMemcpyAsync(e->uniform.p, uniform, s->rows * sizeof(double), cudaMemcpyHostToDevice, e->stream));
        if (const int rs = step_device(e, s, e->tok.as<uint32_t>(), e->logits.as<float>(), nullptr, true)) return rs;
        if (!launch_sample(e->stream, e->logits.as<float>(), s->rows, e->cfg.vocab, temperature, top_k, e->uniform.as<double>(), e->next.as<uint32_t>()))
            return e->fail(AVA_NOT_APPLICABLE, "the sampler does not cover this vocabulary or top_k: pick on the host (ava_step + ava_pick)");
        e->launches++;
        CK(cudaMemcpyAsync(next, e->next.p, s->rows * sizeof(uint32_t), cudaMemcpyDeviceToHost, e->stream));
        return finish(e);
    };
    return txn_end(e, s, txn, body());
}

int ava_forward_with_state(ava_engine* e, ava_state* s, const uint32_t* ids, int32_t t, int32_t last_only, float* logits) {
    int rc = check_pair(e, s);
    if (rc) return rc;
    if (!ids || !logits || t <= 0) return e->fail(AVA_ERR_ARG, "bad arguments");
    const int M = s->rows, V = e->cfg.vocab;
    for (size_t i = 0; i < (size_t)M * t; ++i)
        if (ids[i] >= (uint32_t)V) return e->fail(AVA_ERR_ARG, "token %u outside the vocabulary", ids[i]);
    // the ids column by column: position j of every row is one step
    std::vector<uint32_t> col((size_t)t * M);
    for (int r = 0; r < M; ++r)
        for (int j = 0; j < t; ++j) col[(size_t)j * M + r] = ids[(size_t)r * t + j];
    Txn txn;
    if ((rc = txn_begin(e, s, false, txn))) return rc;
    auto body = [&]() -> int {
    int rc = AVA_OK;
    Dev dcol;
    CK(dcol.alloc(col.size() * sizeof(uint32_t)));
    CK(cudaMemcpyAsync(dcol.p, col.data(), col.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, e->stream));
    // the prompt goes in chunks of Tc tokens per row: token-parallel work over Tc x rows token-rows at once, the
    // recurrences in order inside their kernels (step_device).  The chunk is sized to a bounded work space.
    int64_t max_rows = 16384;
    if (!last_only) max_rows = std::min<int64_t>(max_rows, std::max<int64_t>(M, ((int64_t)1 << 28) / V));  // logits of a chunk <= 1 GiB
    const int Tc = (int)std::max<int64_t>(1, std::min<int64_t>(t, max_rows / M));
    if ((rc = ensure_workspace(e, *e, M * Tc, last_only ? M : M * Tc))) return rc;
    for (int j0 = 0; j0 < t; j0 += Tc) {
        const int T = std::min(Tc, t - j0);
        const bool last_chunk = j0 + T == t;
        const bool want = !last_only || last_chunk;
        if ((rc = step_device(e, s, dcol.as<uint32_t>() + (size_t)j0 * M, want ? e->logits.as<float>() : nullptr, nullptr, want, T, !last_only))) return rc;
        if (!want) continue;
        if (last_only) {
            CK(cudaMemcpyAsync(logits, e->logits.p, (size_t)M * V * sizeof(float), cudaMemcpyDeviceToHost, e->stream));
        } else {
            // device [T][rows][vocab] -> host [rows][t][vocab]: position j0 + k of every row
            for (int k = 0; k < T; ++k)
                CK(cudaMemcpy2DAsync(logits + (size_t)(j0 + k) * V, (size_t)t * V * sizeof(float), e->logits.as<float>() + (size_t)k * M * V,
                                     (size_t)V * sizeof(float), (size_t)V * sizeof(float), M, cudaMemcpyDeviceToHost, e->stream));
            CK(cudaStreamSynchronize(e->stream));  // the logits buffer is reused by the next chunk
        }
    }
    return finish(e);
    };
    return txn_end(e, s, txn, body());
}

int ava_prefill_device(ava_engine* e, ava_state* s, const uint32_t* tok_device, int32_t t, int32_t chunk, float* logits_device, uint32_t* next_device) {
    int rc = check_pair(e, s);
    if (rc) return rc;
    if (!tok_device || t <= 0 || chunk <= 0) return e->fail(AVA_ERR_ARG, "bad arguments");
    const int M = s->rows;
    const int Tc = std::min(chunk, t);
    if ((rc = ensure_workspace(e, *e, M * Tc, M))) return rc;
    for (int j0 = 0; j0 < t; j0 += Tc) {
        const int T = std::min(Tc, t - j0);
        const bool last_chunk = j0 + T == t;
        const bool want = last_chunk && (logits_device || next_device);
        if ((rc = step_device(e, s, tok_device + (size_t)j0 * M, want ? logits_device : nullptr, want ? next_device : nullptr, want && logits_device, T, false)))
            return rc;
    }
    return AVA_OK;
}

// ---- the engram store split by position over several GPUs (one long sequence) ---------------------------------
int ava_state_set_kv_shard(ava_state* s, int32_t rank, int32_t world, int64_t block, int64_t position) {
    if (!s || world < 1 || rank < 0 || rank >= world || block < 1 || position < 0) return AVA_ERR_ARG;
    if (s->e->cfg.eng_block < 0) return s->e->fail(AVA_ERR_ARG, "the model has no engram");
    if (s->e->cfg.eng_cap > 0) return s->e->fail(AVA_NOT_APPLICABLE, "a capped store is not split");
    s->shard_world = world;
    s->shard_rank = rank;
    s->shard_block = block;
    s->shard_pos = position;
    return AVA_OK;
}

int32_t ava_shard_parts(const ava_engine* e, const ava_state* s) {
    if (!e || !s) return -1;
    return engram_segments(s->ring, e->long_seg > 0 ? e->long_seg : 2048);
}

int ava_split_step_begin(ava_engine* e, ava_state* s, const uint32_t* tok_device, float* qkv_device) {
    int rc = check_pair(e, s);
    if (rc) return rc;
    if (!tok_device || !qkv_device || e->cfg.eng_block < 0) return e->fail(AVA_ERR_ARG, "bad arguments");
    // the second half of the step reads the token ids again (the surprise, the cerebellum's input): they are kept
    if (tok_device != e->tok.as<uint32_t>())
        CK(cudaMemcpyAsync(e->tok.p, tok_device, (size_t)s->rows * sizeof(uint32_t), cudaMemcpyDeviceToDevice, e->stream));
    if ((rc = step_device(e, s, e->tok.as<uint32_t>(), nullptr, nullptr, false, 1, false, PHASE_BEGIN))) return rc;
    CK(cudaMemcpyAsync(qkv_device, e->eqkv.p, (size_t)s->rows * 3 * e->cfg.d * sizeof(float), cudaMemcpyDeviceToDevice, e->stream));
    return AVA_OK;
}

int ava_shard_partial(ava_engine* e, ava_state* s, const float* qkv_device, float* partial_device) {
    int rc = check_pair(e, s);
    if (rc) return rc;
    if (!qkv_device || !partial_device || s->shard_world < 1) return e->fail(AVA_ERR_ARG, "the state has no shard set");
    const ava_config& c = e->cfg;
    const int rows = s->rows, d = c.d;
    EngramArgs ea{};
    ea.qkv = qkv_device;
    ea.k = s->eng_k.p; ea.v = s->eng_v.p;
    ea.n = s->eng_n.as<int32_t>(); ea.start = s->eng_start.as<int32_t>();
    ea.M = rows; ea.d = d; ea.hs = c.eng_head_size; ea.cap = s->ring; ea.keep = s->keep; ea.bf16 = c.eng_store_bf16;
    ea.status = e->status.as<uint32_t>();
    const int owner = (int)std::min<int64_t>(s->shard_pos / s->shard_block, s->shard_world - 1);
    if (owner == s->shard_rank) {
        for (int r = 0; r < rows; ++r)
            if (s->n_host[r] >= s->ring) return e->fail(AVA_ERR_CAPACITY, "this rank's part of the engram store is full (%d tokens)", s->ring);
        prof_begin(e, "engram.append");
        launch_engram_append(e->stream, ea);
        prof_end(e);
        e->launches++;
        for (int r = 0; r < rows; ++r) s->n_host[r] += 1;
    }
    s->shard_pos += 1;
    const int seg_len = e->long_seg > 0 ? e->long_seg : 2048;
    const int n_seg = engram_segments(s->ring, seg_len);
    prof_begin(e, "engram.partial");
    if (!launch_engram_partial(e->stream, ea, seg_len, n_seg, partial_device))
        return e->fail(AVA_ERR_CAPACITY, "engram segments of %d keys do not fit shared memory", seg_len);
    prof_end(e);
    cudaError_t le = take_launch_error();
    if (le == cudaSuccess) le = cudaGetLastError();
    if (le != cudaSuccess) return e->cuda_fail(le, "kernel launch");
    return AVA_OK;
}

int ava_split_step_end(ava_engine* e, ava_state* s, const float* gathered_device, int32_t world, float* logits_device, uint32_t* next_device) {
    int rc = check_pair(e, s);
    if (rc) return rc;
    if (!gathered_device || world < 1) return e->fail(AVA_ERR_ARG, "bad arguments");
    const ava_config& c = e->cfg;
    const int seg_len = e->long_seg > 0 ? e->long_seg : 2048;
    prof_begin(e, "engram.combine");
    launch_engram_combine(e->stream, gathered_device, s->rows, c.d / c.eng_head_size, c.eng_head_size, engram_segments(s->ring, seg_len), e->eo.as<float>(), world);
    prof_end(e);
    return step_device(e, s, e->tok.as<uint32_t>(), logits_device, next_device, logits_device != nullptr, 1, false, PHASE_END);
}

void* ava_engine_stream(ava_engine* e) { return e ? (void*)e->stream : nullptr; }
int64_t ava_engine_launches(const ava_engine* e) { return e ? e->launches : 0; }

int64_t ava_engine_bytes(const ava_engine* e) {
    if (!e) return 0;
    int64_t n = e->tok_emb.bytes + e->final_norm.bytes + e->head.q.bytes + e->head.scale.bytes;
    for (const auto& bp : e->blocks) {
        const BlockDev& b = *bp;
        for (const Dev* d : {&b.mem_norm, &b.beta, &b.theta, &b.rho, &b.again, &b.hebb_norm, &b.gate_w, &b.ba, &b.bb, &b.wa2, &b.wb2,
                             &b.off, &b.vres, &b.eng_norm, &b.mlp_norm, &b.dense})
            n += d->bytes;
        for (const QMat* q : {&b.win, &b.wout, &b.proj, &b.wo, &b.eqkv, &b.ewo, &b.w1, &b.w2}) n += q->q.bytes + q->scale.bytes;
    }
    for (const Dev* d : {&e->x, &e->h, &e->proj, &e->ve, &e->vv, &e->vw, &e->vah, &e->vqg, &e->vex, &e->qw, &e->qa, &e->yraw, &e->y, &e->eqkv, &e->eo,
                         &e->u, &e->act, &e->streams, &e->v_first, &e->logits, &e->tok, &e->next})
        n += d->bytes;
    return n;
}

int64_t ava_state_bytes(const ava_state* s) {
    if (!s) return 0;
    int64_t n = 0;
    for (const Dev* d : {&s->lif_v, &s->lif_s, &s->lif_a, &s->mem_f, &s->mem_s, &s->stp_u, &s->stp_x, &s->sur_prev, &s->sur_valid, &s->sur_last, &s->mood, &s->rh, &s->eng_k, &s->eng_v, &s->eng_n, &s->eng_start})
        n += d->bytes;
    return n;
}

int ava_engine_set_segmented_read(ava_engine* e, int32_t seg_len) {
    if (!e || seg_len < 0 || (seg_len > 0 && seg_len < 8)) return AVA_ERR_ARG;
    e->long_seg = seg_len;
    return AVA_OK;
}

const ava_config* ava_engine_config(const ava_engine* e) { return e ? &e->cfg : nullptr; }
int ava_engine_device(const ava_engine* e) { return e ? e->device : -1; }

int ava_engine_set_lanes(ava_engine* e, int32_t lanes) {
    if (!e || lanes < 1 || lanes > 8) return AVA_ERR_ARG;
    e->n_lanes = lanes;
    return AVA_OK;
}

int ava_engine_set_chunked_memory(ava_engine* e, int32_t on) {
    if (!e) return AVA_ERR_ARG;
    e->chunk_mem = on != 0;
    return AVA_OK;
}

int ava_engine_chunked_memory_counts(const ava_engine* e, int64_t* chunked, int64_t* token_loop, int64_t* engram_chunks) {
    if (!e || !chunked || !token_loop || !engram_chunks) return AVA_ERR_ARG;
    *chunked = e->chunked_blocks;
    *token_loop = e->chunk_fallbacks;
    *engram_chunks = e->chunked_reads;
    return AVA_OK;
}

int ava_engine_set_fast_products(ava_engine* e, int32_t on) {
    if (!e) return AVA_ERR_ARG;
    if (!e->finalized) return e->fail(AVA_ERR_ARG, "engine not finalized");
    CK(cudaSetDevice(e->device));
    if (on) {
        // bf16 [dout][din] copies of the matrices (exact: int8 values)
        std::vector<QMat*> mats{&e->head};
        for (auto& b : e->blocks)
            for (QMat* m : {&b->win, &b->wout, &b->proj, &b->wo, &b->eqkv, &b->ewo, &b->w1, &b->w2}) mats.push_back(m);
        for (QMat* m : mats) {
            if (!m->q.p || m->wt.p || m->din % 64 || m->dout % 4) continue;
            CK(m->wt.alloc((size_t)m->din * m->dout * sizeof(uint16_t)));
            launch_widen_transpose(e->stream, m->qp(), m->din, m->dout, m->wt.as<uint16_t>());
        }
        // the gates' first-stage matrix [d][gate_cols] f32, transposed and split into limbs
        for (auto& b : e->blocks) {
            if (!b->gate_w.p || b->gate_wl.p || e->cfg.d % 64) continue;
            const size_t n = (size_t)e->cfg.d * e->gate_cols;
            std::vector<float> hw(n), ht(n);
            CK(cudaMemcpy(hw.data(), b->gate_w.p, n * sizeof(float), cudaMemcpyDeviceToHost));
            for (int k = 0; k < e->cfg.d; ++k)
                for (int c = 0; c < e->gate_cols; ++c) ht[(size_t)c * e->cfg.d + k] = hw[(size_t)k * e->gate_cols + c];
            Dev tmp;
            CK(tmp.alloc(n * sizeof(float)));
            CK(cudaMemcpy(tmp.p, ht.data(), n * sizeof(float), cudaMemcpyHostToDevice));
            CK(b->gate_wl.alloc(3 * n * sizeof(uint16_t)));
            launch_split3(e->stream, tmp.as<float>(), (int64_t)n, b->gate_wl.as<uint16_t>());
            CK(cudaStreamSynchronize(e->stream));
        }
        CK(cudaStreamSynchronize(e->stream));
    }
    e->fast = on != 0;
    return AVA_OK;
}

int ava_debug_keep(ava_engine* e, int32_t on) {
    if (!e) return AVA_ERR_ARG;
    e->keep = on != 0;
    if (!on) e->debug.clear();
    return AVA_OK;
}

int64_t ava_debug_width(const ava_engine* e, const char* name) {
    if (!e || !name) return -1;
    auto it = e->debug_width.find(name);
    return it == e->debug_width.end() ? -1 : it->second;
}

int ava_debug_get(ava_engine* e, const char* name, int32_t block, float* out) {
    if (!e || !name || !out) return AVA_ERR_ARG;
    auto it = e->debug.find({name, block});
    if (it == e->debug.end()) return e->fail(AVA_ERR_ARG, "no kept tensor %s of block %d", name, block);
    CK(cudaSetDevice(e->device));
    CK(cudaStreamSynchronize(e->stream));
    CK(cudaMemcpy(out, it->second->p, it->second->bytes, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

int ava_prof_enable(ava_engine* e, int32_t on) {
    if (!e) return AVA_ERR_ARG;
    CK(cudaSetDevice(e->device));
    CK(cudaStreamSynchronize(e->stream));
    for (auto& p : e->prof_pending) {
        cudaEventDestroy(p.a);
        cudaEventDestroy(p.b);
    }
    e->prof_pending.clear();
    e->prof_total.clear();
    e->prof = on != 0;
    return AVA_OK;
}

int ava_prof_read(ava_engine* e, const char* kernel, int64_t* launches, double* ms) {
    if (!e || !kernel) return AVA_ERR_ARG;
    CK(cudaSetDevice(e->device));
    CK(cudaStreamSynchronize(e->stream));
    for (auto& w : e->more_lanes)
        if (w->lane_stream) CK(cudaStreamSynchronize(w->lane_stream));
    if (const char* path = e->prof_pending.empty() ? nullptr : std::getenv("AVA_TIMELINE")) {  // tuning aid: every bracketed launch with its start and end (ms since the first)
        if (FILE* fp = std::fopen(path, "w")) {
            for (auto& p : e->prof_pending) {
                float t0 = 0.f, t1 = 0.f;
                if (cudaEventElapsedTime(&t0, e->prof_pending.front().a, p.a) == cudaSuccess && cudaEventElapsedTime(&t1, e->prof_pending.front().a, p.b) == cudaSuccess)
                    std::fprintf(fp, "%p %s %.4f %.4f\n", (void*)p.st, p.cls, t0, t1);
            }
            std::fclose(fp);
        }
    }
    for (auto& p : e->prof_pending) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, p.a, p.b) == cudaSuccess) {
            auto& slot = e->prof_total[p.cls];
            slot.first += 1;
            slot.second += t;
        }
        cudaEventDestroy(p.a);
        cudaEventDestroy(p.b);
    }
    e->prof_pending.clear();
    auto it = e->prof_total.find(kernel);
    if (launches) *launches = it == e->prof_total.end() ? 0 : it->second.first;
    if (ms) *ms = it == e->prof_total.end() ? 0.0 : it->second.second;
    return AVA_OK;
}

int ava_prof_names(ava_engine* e, char* out, int32_t cap) {
    if (!e || !out || cap <= 0) return AVA_ERR_ARG;
    std::string all;
    for (auto& p : e->prof_pending) e->prof_total[p.cls];
    for (auto& kv : e->prof_total) all += kv.first + "\n";
    snprintf(out, cap, "%s", all.c_str());
    return AVA_OK;
}

// ---- the split step's exchange behind the boundary: NCCL reached by dlopen, the caller's (or our own) communicator ----
int ava_nccl_version(int32_t* version) {
    const NcclApi* n = nccl_api();
    if (!n || !version) return AVA_NOT_APPLICABLE;
    int v = 0;
    if (n->GetVersion(&v) != 0) return AVA_ERR_CUDA;
    *version = v;
    return AVA_OK;
}

int ava_nccl_unique_id(unsigned char* id128) {
    const NcclApi* n = nccl_api();
    if (!id128) return AVA_ERR_ARG;
    if (!n) return AVA_NOT_APPLICABLE;
    NcclUniqueId id;
    if (n->GetUniqueId(&id) != 0) return AVA_ERR_CUDA;
    std::memcpy(id128, id.internal, 128);
    return AVA_OK;
}

int ava_nccl_comm_init(ava_engine* e, int32_t world, int32_t rank, const unsigned char* id128, void** comm) {
    if (!e || !id128 || !comm || world < 1 || rank < 0 || rank >= world) return AVA_ERR_ARG;
    const NcclApi* n = nccl_api();
    if (!n) return e->fail(AVA_NOT_APPLICABLE, "no NCCL library: %s", nccl_dl_error());
    CK(cudaSetDevice(e->device));
    NcclUniqueId id;
    std::memcpy(id.internal, id128, 128);
    void* c = nullptr;
    const int rc = n->CommInitRank(&c, world, id, rank);
    if (rc != 0) return e->fail(AVA_ERR_CUDA, "ncclCommInitRank: %s", n->GetErrorString(rc));
    *comm = c;
    return AVA_OK;
}

int ava_nccl_comm_destroy(void* comm) {
    const NcclApi* n = nccl_api();
    if (!n || !comm) return AVA_ERR_ARG;
    return n->CommDestroy(comm) == 0 ? AVA_OK : AVA_ERR_CUDA;
}

int ava_split_step(ava_engine* e, ava_state* s, void* nccl_comm, int32_t rank, int32_t world, const uint32_t* tok_device, float* qkv_device,
                   float* partial_device, float* gathered_device, float* logits_device, uint32_t* next_device) {
    int rc = check_pair(e, s);
    if (rc) return rc;
    if (!qkv_device || !partial_device || !gathered_device || world < 1 || rank < 0 || rank >= world || (rank == 0 && !tok_device) || (world > 1 && !nccl_comm))
        return e->fail(AVA_ERR_ARG, "bad arguments");
    const bool use_nccl = nccl_comm != nullptr;  // one rank with a communicator still goes through NCCL
    const NcclApi* n = use_nccl ? nccl_api() : nullptr;
    if (use_nccl && !n) return e->fail(AVA_NOT_APPLICABLE, "no NCCL library: %s", nccl_dl_error());
    const ava_config& c = e->cfg;
    const size_t qkv_n = (size_t)s->rows * 3 * c.d;
    const size_t part_n = (size_t)s->rows * (c.d / c.eng_head_size) * ava_shard_parts(e, s) * (2 + c.eng_head_size);
    if (rank == 0 && (rc = ava_split_step_begin(e, s, tok_device, qkv_device))) return rc;
    if (use_nccl) {
        const int nrc = n->Broadcast(qkv_device, qkv_device, qkv_n, NCCL_FLOAT32, 0, nccl_comm, e->stream);
        if (nrc != 0) return e->fail(AVA_ERR_CUDA, "ncclBroadcast: %s", n->GetErrorString(nrc));
    }
    if ((rc = ava_shard_partial(e, s, qkv_device, partial_device))) return rc;
    if (use_nccl) {
        const int nrc = n->AllGather(partial_device, gathered_device, part_n, NCCL_FLOAT32, nccl_comm, e->stream);
        if (nrc != 0) return e->fail(AVA_ERR_CUDA, "ncclAllGather: %s", n->GetErrorString(nrc));
    } else {
        CK(cudaMemcpyAsync(gathered_device, partial_device, part_n * sizeof(float), cudaMemcpyDeviceToDevice, e->stream));
    }
    if (rank == 0) return ava_split_step_end(e, s, gathered_device, world, logits_device, next_device);
    return AVA_OK;
}

int ava_split_wait(ava_engine* e, void* nccl_comm, int32_t timeout_ms) {
    if (!e || timeout_ms < 0) return AVA_ERR_ARG;
    const NcclApi* n = nccl_comm ? nccl_api() : nullptr;
    if (nccl_comm && !n) return e->fail(AVA_NOT_APPLICABLE, "no NCCL library: %s", nccl_dl_error());
    CK(cudaSetDevice(e->device));
    cudaEvent_t done;
    CK(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
    cudaError_t ce = cudaEventRecord(done, e->stream);
    const auto t0 = std::chrono::steady_clock::now();
    int why = 0;  // 1: NCCL reported an error, 2: the time ran out
    int async_error = 0;
    while (ce == cudaSuccess) {
        ce = cudaEventQuery(done);
        if (ce != cudaErrorNotReady) break;
        ce = cudaSuccess;
        if (n && n->CommGetAsyncError && n->CommGetAsyncError(nccl_comm, &async_error) == 0 && async_error != 0 && async_error != NCCL_IN_PROGRESS) {
            why = 1;
            break;
        }
        if (std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() >= timeout_ms) {
            why = 2;
            break;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (why != 0) {
        // The collective's kernel is waiting for a rank that will not come: only an abort ends it.  The communicator is
        // gone after it, whatever the abort answers.
        const bool aborted = n && n->CommAbort && n->CommAbort(nccl_comm) == 0;
        if (aborted) cudaStreamSynchronize(e->stream);
        cudaEventDestroy(done);
        if (why == 1) return e->fail(AVA_ERR_CUDA, "NCCL: %s%s", n->GetErrorString(async_error), aborted ? " (communicator aborted)" : "");
        return e->fail(AVA_ERR_CUDA, "the split step did not finish within %d ms%s", (int)timeout_ms, aborted ? " (communicator aborted)" : "");
    }
    cudaEventDestroy(done);
    if (ce != cudaSuccess) return e->fail(AVA_ERR_CUDA, "%s", cudaGetErrorString(ce));
    return AVA_OK;
}

float ava_host_expf(float x) { return ava::expf_(x); }
float ava_host_logf(float x) { return ava::logf_(x); }
float ava_host_rsqrtf(float x) { return ava::rsqrtf_(x); }
float ava_host_sinf(float x) { return ava::sinf_(x); }
float ava_host_cosf(float x) { return ava::cosf_(x); }

}  // extern "C"
