/* CPU oracle for the per-token block step of the Ava spiking language model.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker that the CUDA engine is
 * compared with; it is never linked into, loaded by or called from the product
 * library.  Only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg may load it.
 *
 * It restates, in plain sequential C++, the arithmetic of the reference's int8 CPU
 * engine (nochallenge/ava, crate design-tests/nn/gpu), keeping the order of every
 * floating-point operation the reference documents:
 *   quantiser            design-tests/nn/parts/src/quant.rs:18-31
 *   int8 products        design-tests/nn/gpu/src/int8.rs:124-211,315-331 (event rule :10-13,142-147)
 *   norms, gemv, gates   design-tests/nn/gpu/src/model/fstep.rs:200-299
 *   engram read          design-tests/nn/gpu/src/model/fstep.rs:303-356
 *   plain delta rule     design-tests/nn/gpu/src/model/fstep.rs:397-436
 *   LIF (int2, ALIF)     design-tests/nn/gpu/src/model/fstep/arch.rs:173-228
 *   fast-weight head     design-tests/nn/gpu/src/model/fstep/arch.rs:256-337
 *   block wiring         design-tests/nn/gpu/src/model/fstep/arch.rs:525-1073
 *
 * Parity status: the reference cannot be built in this environment (no Rust tool
 * chain, un-vendored crates), so no absolute logits of the author's binary are
 * pinned.  What is pinned are the reference's own hand-worked vectors and the
 * identities its tests assert (see tests/test_oracle_golden.py).  End-to-end
 * numeric parity with the author's binary is therefore "parity unpinned".
 *
 * Transcendentals: the reference takes exp, ln and powf from the platform libm.
 * The oracle defaults to this machine's libm and lets a test plug in other
 * implementations (orc_set_math) so that a device implementation can be compared
 * bit for bit.
 */
#ifndef AVA_ORACLE_H
#define AVA_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct orc_config {
    int32_t vocab;
    int32_t d;              /* model width */
    int32_t n_blocks;
    int32_t hidden;         /* wide layer (4 d in the reference) */
    int32_t kwta_k;         /* units the k-winners-take-all keeps */
    int32_t head_size;      /* fast-weight memory head size; heads = d / head_size */
    int32_t eng_block;      /* block that holds the engram read; -1: none */
    int32_t eng_head_size;  /* engram head size (32 in the reference) */
    int32_t eng_store_bf16; /* 1: keys/values rounded to bf16 when stored */
    int32_t eng_cap;        /* oldest-first cap on stored tokens; 0: none */
    int32_t gate_rank;      /* rank of the per-channel gates' low-rank projections */
    int32_t spikes;         /* 0 binary, 1 ternary, 2 int2 */
    int32_t alif;           /* adaptive threshold trace */
    int32_t theta;          /* per-neuron thresholds given (else 1.0) */
    int32_t lif_scale;      /* input current times (1 - beta) */
    int32_t value_residual;
    int32_t relu2;          /* square the kept MLP units */
    int32_t dense;          /* dense residual mixes */
    int32_t out_gate;       /* 1: silu(h Wg) output gate on the memory read */
    int32_t fast_mem;       /* 1: blocks have the fast-weight memory; 0: kind S (src/model/fstep.rs:461-688) */
    int32_t dendrite;       /* --dendrite: MLP units times 1 + tanh(head_norm(memory read) A B) (fstep/arch_f4.rs:120-141) */
    int32_t neuromod;       /* --neuromod k (3): NE, ACh, DA signals from a nucleus after block 0 (src/v50.rs:20-29) */
    int32_t stp;            /* --stp: the spikes reach W_out through a short-term-plastic synapse (fstep/arch_f3.rs:72-106) */
    int32_t dopamine;       /* --dopamine: the surprise at this token scales the later blocks' MLP output (fstep/arch_f4.rs:131-143) */
    int32_t mood;           /* --mood (4 units): a slow trace of the surprise scales the later blocks' LIF current (fstep/arch_f3.rs:106-186) */
    int32_t cb_units;       /* --cerebellum-head G: G sparse granule units correct the final normed state (fstep/arch_f3.rs:207-283) */
    int32_t letters;        /* --letters: each token's spelling adds a vector to its input (fstep/arch_f2.rs:34-60) */
    int32_t rhythm;         /* --rhythm: two resettable clocks' phases scale the memory's write strength and read per head (fstep/arch_f4.rs:39-108) */
    int32_t thalamus;       /* --thalamus: a relay reads the stream and gates each block's memory read and residual (fstep/arch_f2.rs:62-153) */
    float   mem_momentum;   /* 0: off */
    float   slope;          /* surrogate slope (forward value cancels; kept for the literal op order) */
} orc_config;

typedef float (*orc_fn1)(float);

/* Replace exp / ln / x^-0.5 (NULL keeps the current one).  Process-wide. */
void orc_set_math(orc_fn1 expf_, orc_fn1 logf_, orc_fn1 rsqrtf_);
void orc_reset_math(void);
/* Replace sine and cosine (--rhythm's phases; NULL keeps the current one).  orc_reset_math puts the platform's back. */
void orc_set_trig(orc_fn1 sinf_, orc_fn1 cosf_);
void orc_set_threads(int n);
/* 1: AVX2+FMA tile kernel for the int8 products (same bits as scalar); 0: scalar. */
void orc_set_simd(int on);
/* share of non-zero inputs at or below which a row runs as an event sum; <0 never */
void orc_set_event_max(double v);

/* ---- op level -------------------------------------------------------------- */
/* A0: symmetric per-output-column int8. w [rows, cols] row-major. */
void orc_quantize_int8(const float* w, int rows, int cols, int8_t* q, float* scale);
/* A1: y [m, dout] = x [m, din] . (q [din, dout] row-major int8, scale [dout]). */
void orc_q8_matmul(const float* x, int m, const int8_t* q, const float* scale, int din, int dout, float* y);
/* number of rows of the last orc_q8_matmul that ran as event sums */
int orc_last_event_rows(void);
void orc_rmsnorm(const float* x, const float* gain, int n, float* y);
void orc_l2_heads(float* x, int n, int hs);
void orc_head_norm(float* y, int n, int hs);
float orc_sigmoid(float x);
float orc_log_sigmoid(float x);
void orc_gemv(const float* x, int k, const float* w, int n, float* out);
/* A3: one LIF update of d channels. theta, rho, gain, a0, a1 may be NULL. */
void orc_lif(const float* cur, const float* beta, const float* theta, const float* rho, const float* gain,
             int spikes, float slope, const float* v0, const float* s0, const float* a0, int d, float* s1,
             float* v1, float* a1);
/* S (--stp): the spikes through the short-term-plastic synapse (fstep/arch_f3.rs:72-106, nn/parts/src/stp.rs:42-85):
 * out [d] what reaches W_out, (u1, x1) the synapse's new state, eff (may be NULL) the efficacy e / U.  The parameters
 * are the raw ones (their sigmoids are taken inside). */
/* --cerebellum-head's wiring for `inputs` inputs and g units of fan-in 4 from the reference's seed: idx [g * 4], w [g * 4] */
void orc_cb_wiring(int inputs, int g, uint32_t* idx, float* w);
void orc_stp(const float* s, const float* u_param, const float* f_param, const float* d_param, const float* mix, const float* u0, const float* x0,
             int d, float* out, float* u1, float* x1, float* eff);
float orc_kth_largest(const float* u, int n, int k);
/* A7: a = max(u * [u - kth >= 0], 0), squared when relu2. */
void orc_kwta(const float* u, int n, int k, int relu2, float* a);
/* A8: one head's read over n keys/values of hs. */
void orc_attend(const float* q, const float* kc, const float* vc, int n, int hs, float scale, float* out);
/* A5: one fast-weight head, the Ava 0.4 form.  s0/s1/qs/p2 NULL without momentum. */
void orc_head_rows(int hs, const float* e, const float* v, const float* w, const float* ah, const float* qg,
                   const float* ex, float qw, float qa, float ke, float tinv, float mom, const float* qs,
                   const float* p2, const float* f0, const float* s0, float* y, float* f1, float* s1);
/* A6: one head of the plain delta rule: F' = ((F - (k p^T) b) al) + (k v^T) b, y = q^T F'. */
void orc_delta_plain(int hs, const float* f0, const float* k, const float* v, const float* q, float al, float b,
                     float* f1, float* y);
/* float -> bf16 -> float, round to nearest even */
float orc_bf16_round(float x);

/* ---- model level ------------------------------------------------------------ */
typedef struct orc_model orc_model;
typedef struct orc_state orc_state;

orc_model* orc_model_new(const orc_config* cfg);
void orc_model_free(orc_model* m);
/* f32 tensor by its reference name ("tok_emb", "b3.mem.beta", "final.norm", ...). Returns 0, or -1 (unknown / size). */
/* --letters: the spelling of every token, bytes[offsets[t] .. offsets[t + 1]) for t in 0 .. vocab - 1 */
int orc_model_set_token_bytes(orc_model* m, const uint8_t* bytes, const int64_t* offsets);
int orc_model_set_f32(orc_model* m, const char* name, const float* data, int64_t n);
/* an int8 matrix [din, dout] with its per-output scales, by name ("b3.hebb.wq", "head"). */
int orc_model_set_q8(orc_model* m, const char* name, const int8_t* q, const float* scale, int din, int dout);
/* an f32 matrix [din, dout]: quantised with A0 and stored as int8 ("head" takes tok_emb^T itself). */
int orc_model_set_q8_from_f32(orc_model* m, const char* name, const float* w, int din, int dout);
/* 0 when every tensor the configuration needs is there; else -1 and the first missing name in `missing`. */
int orc_model_check(orc_model* m, char* missing, int cap);

orc_state* orc_state_new(const orc_model* m, int rows);
void orc_state_free(orc_state* s);
int orc_state_rows(const orc_state* s);
/* rows idx[0..n) of s as a new state (repeats allowed: a fork) */
orc_state* orc_state_select(const orc_state* s, const int32_t* idx, int n);
/* number of floats of a state tensor of row r ("lif.3.v", "lif.3.s", "lif.3.a", "mem.3.f", "mem.3.s",
 * "eng.k", "eng.v" as [heads, n, hs]); -1 unknown */
int64_t orc_state_len(const orc_state* s, int row, const char* name);
int orc_state_get(const orc_state* s, int row, const char* name, float* out);
int orc_state_put(orc_state* s, int row, const char* name, const float* in, int64_t n);
int64_t orc_state_seen(const orc_state* s, int row);

/* One token per row.  logits [rows, vocab].  Returns 0; 1 when a non-finite gate/key made the reference's
 * fused step refuse the token (the state of that row is then left untouched); <0 on error. */
int orc_step(const orc_model* m, orc_state* s, const uint32_t* tok, float* logits);
/* ids [rows, t] row-major, token by token.  logits [rows, t, vocab], or with last_only [rows, vocab]. */
int orc_forward(const orc_model* m, orc_state* s, const uint32_t* ids, int t, int last_only, float* logits);

/* Per-block intermediates of the last orc_step (row 0 only), for teacher-forced checks:
 * "h_lif","cur","spikes","x_lif","h_mem","qkveg","q","k","v","ek","w","ah","qg","ex","qw","qa","y_raw","y",
 * "x_mem","h_eng","eng_qkv","eng_o","x_eng","h_mlp","u","a","x_out" (block >= 0) and "x_final","x_in" (block -1). */
int64_t orc_trace_len(const char* name, int block);
int orc_trace_get(const char* name, int block, float* out);
void orc_trace_enable(int on);

/* ---- the chunk-parallel forms of the fast-weight memory (ava_chunk.cpp), one head each ------------------------------
 * (I + A)^-1 of a strictly lower-triangular A [c, c] by block doubling (src/model.rs:720-742). */
void orc_inv_unit_lower(const float* a, int c, float* t);
/* The plain (v0.2) delta rule in its chunk-64 WY form (src/model.rs:744-799): q, k, v [t, hs], log alpha and beta [t],
 * f0 [hs, hs] or NULL; y [t, hs], f1 [hs, hs]. */
void orc_delta_rule_from(int t, int hs, const float* q, const float* k, const float* v, const float* la, const float* beta, const float* f0,
                         float* y, float* f1);
/* The Ava-0.4 rule token by token (src/arch.rs:1091-1136): q, k, e, v [t, hs]; la, b [t, g] (g 1 or hs); momentum m;
 * f0, s0 [hs, hs] or NULL; cap bounds the state (1e5 in the reference).  y [t, hs], f1, s1 [hs, hs] (s1 may be NULL). */
void orc_delta_rec(int t, int hs, int g, const float* q, const float* k, const float* e, const float* v, const float* la, const float* b, float m,
                   const float* f0, const float* s0, float cap, float* y, float* f1, float* s1);
/* The same rule in chunks (src/arch.rs:1151-1173, 1243-1327), same arguments without the cap. */
void orc_delta_chunk(int t, int hs, int g, const float* q, const float* k, const float* e, const float* v, const float* la, const float* b, float m,
                     const float* f0, const float* s0, float* y, float* f1, float* s1);

#ifdef __cplusplus
}
#endif
#endif
