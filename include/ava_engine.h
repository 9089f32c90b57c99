/* ava_engine.h — C ABI of the B200 engine for Ava's per-token block step.
 *
 * The reference (nochallenge/ava, crate design-tests/nn/gpu) has no FFI of its own: its seams are Rust-internal.
 * Each entry point below names the reference interface it stands in for (file:line inside the reference project),
 * so that a Rust `extern "C"` block can bind them one to one (bindings/ava_engine.rs is that block).
 *
 * Conventions
 *   - plain pointers and sizes only; every buffer is HOST memory unless the name says `_device`;
 *   - return value: 0 = done; 1 = AVA_NOT_APPLICABLE, the reference's `Ok(None)` convention ("this fast path does not
 *     cover the model or state as it is set; nothing was changed", src/model/fstep.rs:61-101, fstep/arch.rs:42-129);
 *     < 0 = error, text in ava_last_error();
 *   - one host thread drives an engine (the reference's `Model` is !Sync, src/model.rs:398-423); the engine owns its
 *     CUDA stream; states belong to the engine that made them;
 *   - the library has no CPU fallback: without a CUDA device every compute call fails with AVA_ERR_CUDA.
 */
#ifndef AVA_ENGINE_H
#define AVA_ENGINE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AVA_OK 0
#define AVA_NOT_APPLICABLE 1
#define AVA_ERR_ARG (-1)
#define AVA_ERR_CUDA (-2)
#define AVA_ERR_STATE (-3)
#define AVA_ERR_NONFINITE (-4)
#define AVA_ERR_MISSING (-5)
#define AVA_ERR_CAPACITY (-6)

/* Shape and block options: the fields of the reference's `Config` (src/model.rs:158-177) and of `Arch`
 * (src/arch.rs:149-197) that the one-token step reads. */
typedef struct ava_config {
    int32_t vocab;
    int32_t d;              /* model width */
    int32_t n_blocks;
    int32_t hidden;         /* wide layer */
    int32_t kwta_k;         /* units the k-winners-take-all keeps (hidden / kwta_div, src/model.rs:265-267) */
    int32_t head_size;      /* fast-weight memory head size (--head-size); heads = d / head_size */
    int32_t eng_block;      /* block with the engram read (Config::engram); -1: none */
    int32_t eng_head_size;  /* engram head size (HEAD_SIZE = 32 in the reference, src/model.rs:43) */
    int32_t eng_store_bf16; /* 1: keys and values are stored as bf16 (the reference stores f32) */
    int32_t eng_cap;        /* EngramCap { max, rule: Oldest } (src/state.rs:46-49); 0: no cap */
    int32_t gate_rank;      /* GATE_RANK (src/arch.rs:80) */
    int32_t spikes;         /* Spikes: 0 binary, 1 ternary, 2 int2 */
    int32_t alif;           /* --alif */
    int32_t theta;          /* per-neuron thresholds present (--homeostasis) */
    int32_t lif_scale;      /* --lif-scale */
    int32_t value_residual; /* --value-residual */
    int32_t relu2;          /* --mlp-act relu2 */
    int32_t dense;          /* --residual dense */
    int32_t out_gate;       /* 1: silu(h Wg) output gate (OutGate::Silu) */
    int32_t fast_mem;       /* 1: every block has the fast-weight memory (Kind::D / A, src/model.rs:110-118); 0: Kind::S,
                               the spiking memory and the sparse MLP only (the step of src/model/fstep.rs:461-688) */
    int32_t dendrite;       /* --dendrite: each MLP unit times 1 + tanh(head_norm(c) A B), c the block's memory read after W_o
                               (src/model/fstep/arch_f4.rs:120-141, src/v51.rs:8-10) */
    int32_t neuromod;       /* --neuromod k (2..4; Ava 0.4: 3): a nucleus reads block 0's output and sends every later block three
                               signals 2 sigmoid(.): NE scales the LIF's input current, ACh the memory's write strength (kept in
                               [0, 2]), DA the MLP's output (src/v50.rs:20-29, src/model/fstep/arch.rs:616-651,765,996,1029) */
    int32_t stp;            /* --stp: the spikes reach W_out through a short-term-plastic synapse with carried (u, x)
                               (src/model/fstep/arch_f3.rs:72-106, nn/parts/src/stp.rs) */
    int32_t thalamus;       /* --thalamus: a relay sums 16-wide reads rmsnorm(x) R_j of the blocks' input and of every block's
                               output; block i's two gates 2 sigmoid(tanh(sum / sqrt(reads)) G_i + c_i) scale its memory read
                               and its whole change of the stream (src/model/fstep/arch_f2.rs:62-153, src/v51b.rs:312-325);
                               weights th.read [blocks, d, 16], th.gate [blocks, 16, 2], th.bias [blocks, 2]; needs fast_mem */
    int32_t dopamine;       /* --dopamine: after block 0 the surprise at this token, s = CE(head(prev), token) with prev block 0's
                               normed output at the token before (0 at the start of a stream), z = s / ln(vocab); every later
                               block's MLP output times 1 + tanh(z w + c) per channel, before --neuromod's DA
                               (src/model/fstep/arch_f3.rs:106-150, arch_f4.rs:131-143); weights b{i}.v51.da_w / da_c [d], i > 0;
                               carried per row: v51.prev [d], v51.pvalid [1], v51.last_s [1] */
    int32_t mood;           /* --mood (4 units; --mood-units k): m = (z win + bin) sigmoid(-lam) + m exp(log_sigmoid(lam)) after
                               block 0; every later block's LIF current times 1 + tanh(m G) per channel, after --neuromod's NE
                               (src/model/fstep/arch_f3.rs:150-186); weights v51.mood.lam / win / bin [k], b{i}.v51.mood_g [k, d],
                               i > 0; carried per row: v51.mood [k] (and the surprise's three tensors) */
    int32_t cb_units;       /* --cerebellum-head G (a multiple of 32; Ava 0.4: 12288): G granule units each sum 4 fixed inputs of
                               [final normed state, rmsnorm(the token's embedding)] with weights +-1/2 (wiring from the
                               reference's seed), the top G/32 are kept, rectified and brought to unit length, and their rows of
                               cbh.wo [G, d], summed in unit order, are added to the final normed state before the head
                               (src/model/fstep/arch_f3.rs:207-283, src/v51b.rs:241-266,327-360) */
    int32_t letters;        /* --letters: a token's input also takes l Wo, l the mean-like sum over up to 16 of its bytes of
                               tanh(byte[b] + end[place from the end] + pos[place]) / sqrt(bytes used) (64 wide; src/v51.rs:492-501,
                               src/model/fstep/arch_f2.rs:34-60); weights v51.letters.byte [256, 64] / .pos [16, 64] / .end [16, 64] /
                               .wo [64, d] and the tokens' spellings (ava_engine_set_token_bytes) */
    int32_t rhythm;         /* --rhythm: two clocks count the tokens since their last reset (reset read from the input: time =
                               (1 - reset)(1 + time)), their phases time * exp(lw) give four features cos / sin, and every block's
                               write strength (before ACh's clamp) and head-normed read (before the output gate) are scaled per head
                               by 1 + tanh(f G) (src/model/fstep/arch_f4.rs:39-108); weights v51.rhythm.lw / br [2], .wr [d, 2],
                               b{i}.v51.rh_w / rh_r [4, heads]; carried per row: v51.rh [2]; needs fast_mem.  Sine and cosine are
                               the library's own (ava_host_sinf / ava_host_cosf), the same bits on host and device */
    float   mem_momentum;   /* --mem-momentum (0: off) */
    float   slope;          /* --surrogate-slope (does not change forward values) */
} ava_config;

typedef struct ava_engine ava_engine;
typedef struct ava_state ava_state;

/* ---- model ------------------------------------------------------------------------------------------------ */

/* `Model::new` for inference (src/model.rs:805-918): an engine for this configuration on CUDA device `device`. */
int ava_engine_create(const ava_config* cfg, int device, ava_engine** out);
void ava_engine_destroy(ava_engine* e);
/* Text of the last error of this engine (never NULL). `e` NULL: the last error of engine creation on this thread. */
const char* ava_last_error(const ava_engine* e);

/* Weights by the reference's tensor names (src/model.rs:805-918, src/arch.rs:809-886): "tok_emb" [vocab, d],
 * "final.norm" [d], "b{i}.mem.{norm,beta,theta,arho,again}" [d], "b{i}.hebb.{norm,off}" [d], "b{i}.hebb.{wa,wb}"
 * [d, heads], "b{i}.hebb.{ba,bb}" [heads], "b{i}.hebb.{wa1,wb1}" [d, rank], "b{i}.hebb.{wa2,wb2}" [rank, d],
 * "b{i}.hebb.vres" [2], "b{i}.eng.norm", "b{i}.mlp.norm" [d], "b{i}.dense" [i + 2].  `n` = number of floats. */
int ava_engine_set_f32(ava_engine* e, const char* name, const float* data, int64_t n);
/* --letters: the spelling of every token, bytes[offsets[t] .. offsets[t + 1]) for t in 0 .. vocab - 1 (offsets[0] = 0; vocab + 1
 * offsets).  The reference reads them from its tokenizer's merge file (src/v51.rs:449-469, `set_letters_from_bpe`); here the
 * host that owns the tokenizer passes them in, before ava_engine_finalize. */
int ava_engine_set_token_bytes(ava_engine* e, const uint8_t* bytes, const int64_t* offsets);
/* An int8 matrix W [din, dout] row-major (applied x . W) with one f32 scale per output column — the product of
 * `Model::set_int8` (src/model.rs:949-991) given directly: "b{i}.mem.{win,wout}", "b{i}.hebb.{wq,wk,wv,we,wg,wo}",
 * "b{i}.eng.{wq,wk,wv,wo}", "b{i}.mlp.{w1,w2}", "head" [d, vocab]. */
int ava_engine_set_q8(ava_engine* e, const char* name, const int8_t* q, const float* scale, int32_t din, int32_t dout);
/* The same from f32 weights: quantised as `ava_parts::quant::quantize_int8` does (nn/parts/src/quant.rs:18-31). */
int ava_engine_set_q8_from_f32(ava_engine* e, const char* name, const float* w, int32_t din, int32_t dout);
/* `Model::set_int8(true)` + `set_fused(true)`: checks that every tensor is there, builds the output head from
 * tok_emb^T when none was given (src/int8.rs:82-84), lays the weights out in device memory.  AVA_NOT_APPLICABLE when
 * the configuration has an option the engine does not cover (`Model::fused_blocker`, src/model/fstep.rs:61-101). */
int ava_engine_finalize(ava_engine* e);
/* `Model::fused_blocker`: why the engine does not cover this configuration, or NULL. */
const char* ava_engine_blocker(const ava_engine* e);

/* ---- carried state (src/state.rs:94-116) --------------------------------------------------------------------- */

/* `Model::state(rows)` (src/state.rs:593): zero membranes, spikes, traces and fast weights, empty engram store with
 * room for `max_ctx` tokens per row (the oldest-first cap, when set, bounds it instead). */
int ava_state_new(ava_engine* e, int32_t rows, int32_t max_ctx, ava_state** out);
void ava_state_destroy(ava_state* s);
int32_t ava_state_rows(const ava_state* s);
/* `State::select` (src/state.rs:129-203): rows idx[0..n) as a new state; a repeated row is a fork. */
int ava_state_select(const ava_state* s, const int32_t* idx, int32_t n, ava_state** out);
/* `State::cat` (src/state.rs:207-328): the rows of `parts` one after another as a new state. */
int ava_state_cat(const ava_state* const* parts, int32_t n, ava_state** out);
/* Tokens row `row` has read (`State::seen`). */
int64_t ava_state_seen(const ava_state* s, int32_t row);
/* Tensors of one row by the reference's saved-state names (src/state.rs:1150-1202): "lif.{i}.v|s|a" [d],
 * "mem.{i}.f|s" [heads, hs, hs], "eng.k|v" [eng heads, n, eng hs] (f32 values; a bf16 store is widened). */
int64_t ava_state_len(const ava_state* s, int32_t row, const char* name);
int ava_state_export(const ava_state* s, int32_t row, const char* name, float* out);
int ava_state_import(ava_state* s, int32_t row, const char* name, const float* in, int64_t n);

/* ---- the hot path --------------------------------------------------------------------------------------------- */

/* `Model::step(&mut Stream, tok)` (src/model.rs:1260-1272 -> fstep::arch::step, src/model/fstep/arch.rs:478) for every
 * row of `s` at once: one token per row, logits [rows, vocab].  The rows are independent (src/state.rs:13-15). */
int ava_step(ava_engine* e, ava_state* s, const uint32_t* tok, float* logits);
/* The same, returning only each row's greedy next token (lowest index on ties). */
int ava_step_greedy(ava_engine* e, ava_state* s, const uint32_t* tok, uint32_t* next);
/* `Model::forward_with_state(ids [rows, t], &mut State)` (src/state.rs:684): t tokens per row.  logits [rows, t,
 * vocab], or [rows, vocab] of the last position when last_only (what `Model::feed` keeps, src/model.rs:1218-1227). */
int ava_forward_with_state(ava_engine* e, ava_state* s, const uint32_t* ids, int32_t t, int32_t last_only, float* logits);

/* Commit at the end, as the reference has it (src/model/fstep/arch.rs:1059-1069: the State moves on only once everything
 * is computed; a refusal at :780-783, 861-864 leaves nothing changed).  The kernels update the carried state as they go;
 * with this set (off by default), ava_step, ava_step_greedy, ava_step_sample and ava_forward_with_state put the state
 * back as it was when they fail after work was queued (AVA_ERR_NONFINITE, a full engram store, a wait that ran out): the
 * small carried tensors are copied aside before the call; the fast weights are not copied for a one-token step: the
 * streaming pass reads one copy and writes a second, and the two change places on success (no extra traffic, twice the
 * fast-weight memory).  A prompt, or a memory with momentum, works in place and copies the fast weights aside whole
 * for the call.  The device-queued calls (ava_step_device, ava_prefill_device) report no status and commit as they go. */
int ava_state_set_commit_at_end(ava_state* s, int32_t on);

/* Device-resident forms for callers that keep tokens and logits in GPU memory (no host copies, no synchronise):
 * tok_device [rows] u32, logits_device [rows, vocab] f32 or NULL, next_device [rows] u32 or NULL.  Work is queued on
 * the engine's stream; ava_sync waits for it and returns the step's status. */
int ava_step_device(ava_engine* e, ava_state* s, const uint32_t* tok_device, float* logits_device, uint32_t* next_device);
/* Prompt reading with device-resident ids (`Model::feed`, src/model.rs:1218-1227, without host copies): tok_device
 * [t][rows] u32 (time-major), processed `chunk` tokens per row at a time; logits_device [rows, vocab] and next_device
 * [rows] (either may be NULL) receive the last position's logits / greedy token.  Queued on the engine's stream. */
int ava_prefill_device(ava_engine* e, ava_state* s, const uint32_t* tok_device, int32_t t, int32_t chunk, float* logits_device, uint32_t* next_device);
int ava_sync(ava_engine* e);
/* The engine's cudaStream_t (for timing with CUDA events on the launching stream). */
void* ava_engine_stream(ava_engine* e);
/* Kernels launched by this engine since it was made. */
int64_t ava_engine_launches(const ava_engine* e);
/* Bytes of device memory the engine (weights, work buffers) and a state hold. */
int64_t ava_engine_bytes(const ava_engine* e);
int64_t ava_state_bytes(const ava_state* s);

/* No counterpart in the reference (its engram read materialises all scores on the CPU, src/memory.rs:664-692).  A
 * store too long for one block's shared memory (about 14 k tokens at 12 heads of 64) is read in segments whose partial
 * softmax statistics (max, sum, mix) are merged afterwards; seg_len > 0 makes every read take that path with segments
 * of seg_len keys (0: only when it must).  The segmented read agrees with the one-pass read to rounding, not bit for
 * bit. */
int ava_engine_set_segmented_read(ava_engine* e, int32_t seg_len);

/* No counterpart in the reference (its step runs one row on the host's threads).  A decode step of a large batch runs
 * as `lanes` lanes (1..8, default 2): contiguous windows of the state's rows, each with work buffers and a stream of its
 * own, forked from and joined back into the engine's stream, so that one lane's state pass (HBM-bound) runs beside the
 * other lanes' products (bound by latency).  Rows are independent (src/state.rs:13-15): the bits do not depend on it. */
int ava_engine_set_lanes(ava_engine* e, int32_t lanes);
/* Fast products (no counterpart in the reference; off by default).  on != 0: the dense int8-weight products of the step
 * (W_in, the q|k|v|e|g projection, W_o, the engram's projections, W_1 and the output head) run on the tensor cores:
 * every product exact (the f32 activation as three bf16 limbs, the int8 weight exact in bf16), the f32 sum in the
 * tensor core's order instead of k = 0, 1, ...  The step's results then agree with the reference's to about 1e-6 of
 * each sum's magnitudes instead of bit for bit, and a membrane within that distance of its threshold can spike
 * differently.  In a decode step W_out and W_2 keep the exact event sum; over a prompt chunk of 1024 token-rows or more
 * W_2 is multiplied densely on the tensor cores too, and W_out (rows of spikes: small integers) with one bf16 limb each
 * side, which is exact (integer partial sums below 2^24): that product is still the event sum's bits.  Costs 2 bytes per dense weight of
 * device memory on first use.  Call after ava_engine_finalize, between steps. */
int ava_engine_set_fast_products(ava_engine* e, int32_t on);
/* With fast products on, a prompt chunk reads its two recurrent memories in chunk-parallel forms on the tensor cores
 * (on = 0 keeps the token loops; default on):
 *   the fast-weight memory, when the chunk's length is a multiple of 64, the head size a multiple of 128 and there is no
 *     momentum: `delta_chunk` (design-tests/nn/gpu/src/arch.rs:1151-1173, 1243-1327), which agrees with the token loop
 *     to rounding (the reference's bound for it: 1e-4 of max(1, max|ref|)); a block whose rates forget faster than e^-60
 *     inside 64 tokens falls back to the token loop for that chunk;
 *   the engram, when its head size is 64, the store is bf16 and neither wraps nor trims inside the chunk: the chunk's
 *     keys and values join the store, then one causal pass reads every token (no counterpart in the reference, which
 *     reads once per token: src/model/fstep.rs:303-356); agrees with the one-token read to rounding.
 * ava_engine_chunked_memory_counts reports, since the engine was made, the (block, chunk) passes of the fast-weight memory
 * that took the chunk form and that fell back, and the chunks whose engram read took the causal pass. */
int ava_engine_set_chunked_memory(ava_engine* e, int32_t on);
int ava_engine_chunked_memory_counts(const ava_engine* e, int64_t* chunked, int64_t* token_loop, int64_t* engram_chunks);

/* ---- one long sequence with its engram store split by position over several GPUs ------------------------------
 * No counterpart in the reference (one device, src/memory.rs:664-692).  Each GPU runs one process with its own engine
 * and a state whose store keeps only the tokens it owns: position p belongs to rank min(p / block, world - 1).  The
 * membranes and fast weights are stepped on rank 0 only.  Per token:
 *   rank 0     ava_split_step_begin   blocks up to the engram's q,k,v; copies them [rows, 3 d] to qkv_device
 *   (caller)   broadcast qkv from rank 0 (NCCL)
 *   all ranks  ava_shard_partial      the owner appends k,v; every rank leaves the partial softmax statistics of its
 *                                     part: [rows][heads][ava_shard_parts()][2 + head size] f32 (max, sum, mix)
 *   (caller)   all-gather the partials (NCCL) into [world][...]
 *   rank 0     ava_split_step_end     merges them in position order and finishes the step
 * The merged read agrees with the one-pass read to rounding (the additions are grouped differently), not bit for bit.
 * Every pointer is device memory; work is queued on the engine's stream (the caller orders its NCCL calls after it). */
int ava_state_set_kv_shard(ava_state* s, int32_t rank, int32_t world, int64_t block, int64_t position);
int32_t ava_shard_parts(const ava_engine* e, const ava_state* s);
int ava_split_step_begin(ava_engine* e, ava_state* s, const uint32_t* tok_device, float* qkv_device);
int ava_shard_partial(ava_engine* e, ava_state* s, const float* qkv_device, float* partial_device);
int ava_split_step_end(ava_engine* e, ava_state* s, const float* gathered_device, int32_t world, float* logits_device, uint32_t* next_device);

/* The same token as ONE call, the two collectives included: rank 0 runs ava_split_step_begin, q,k,v are broadcast from
 * rank 0, every rank runs ava_shard_partial, the partials are all-gathered, rank 0 runs ava_split_step_end; all of it
 * queued on the engine's stream.  nccl_comm is an ncclComm_t of `world` ranks whose rank numbers are the shard's (the
 * caller's own communicator, or one made by ava_nccl_comm_init); NCCL is reached with dlopen at the first call
 * (libnccl.so.2, or the library AVA_NCCL_LIB names), the engine's library does not link against it.  The buffers are the
 * caller's device memory: qkv [rows, 3 d], partial [rows][heads][ava_shard_parts()][2 + head size], gathered `world`
 * times that; tok_device, logits_device and next_device are read on rank 0 only.  world == 1 needs no communicator
 * (NULL: the gather is a copy; given one, the two collectives run through it all the same).
 * AVA_NOT_APPLICABLE when no NCCL library can be loaded.
 * ava_nccl_unique_id fills 128 bytes on one rank (the caller carries them to the others by any means it has);
 * ava_nccl_comm_init makes the communicator on the engine's device; ava_nccl_version reports the loaded library's. */
int ava_split_step(ava_engine* e, ava_state* s, void* nccl_comm, int32_t rank, int32_t world, const uint32_t* tok_device, float* qkv_device,
                   float* partial_device, float* gathered_device, float* logits_device, uint32_t* next_device);
int ava_nccl_unique_id(unsigned char* id128);
int ava_nccl_comm_init(ava_engine* e, int32_t world, int32_t rank, const unsigned char* id128, void** comm);
int ava_nccl_comm_destroy(void* comm);
int ava_nccl_version(int32_t* version);

/* A bounded host wait for what is queued on the engine's stream (the split step's collectives among it): returns AVA_OK
 * once the stream has drained.  While it waits it asks NCCL for the communicator's asynchronous error
 * (ncclCommGetAsyncError); on an error, or when timeout_ms have passed (a rank that never joined its collective), it
 * aborts the communicator (ncclCommAbort, which ends the collective's kernel in flight), drains the stream and returns
 * AVA_ERR_CUDA with the reason in ava_last_error: the communicator must not be used or destroyed afterwards, the engine
 * and the state stay usable.  nccl_comm NULL: the same wait without the NCCL queries.  The reference has no
 * counterpart (its sequence never leaves one device). */
int ava_split_wait(ava_engine* e, void* nccl_comm, int32_t timeout_ms);

/* One traced token of a one-row state: `Model::step_trace` (src/model.rs, record built in src/model/fstep/arch.rs:420-476,
 * the chat app's event feed).  The step is the plain one (same logits, same state); the record holds copies of what it
 * computed and sizes taken from those copies on the host.  ava_trace_get(name, block): per block "spikes" [d] as they reach
 * W_out, "winners" [hidden] 0/1, "hidden" [hidden] as it reaches W2, and per memory head "mem_write" (|F' - alpha F|),
 * "mem_read" (|y| before its norm), "mem_keep" (mean alpha), "mem_gate" (mean write strength); at the engram's block
 * "engram_attn" [heads, keys] (this token's key last) and "engram_read" [d]; block -1 "input_rms" [1].  Returns the
 * value count (copying up to cap floats when out is not NULL) or -1.  AVA_NOT_APPLICABLE with a capped engram store. */
typedef struct ava_trace ava_trace;
int ava_step_trace(ava_engine* e, ava_state* s, uint32_t tok, float* logits, ava_trace** out);
int64_t ava_trace_get(const ava_trace* t, const char* name, int32_t block, float* out, int64_t cap);
void ava_trace_free(ava_trace* t);

/* Section clock, as the reference's fused step keeps one (`take_secs`, src/model/fstep/arch.rs:131-165, switched by
 * `int8::set_mm_prof`, src/int8.rs:635-640): with it on, every kernel launch is bracketed by CUDA events on the
 * engine's stream.  ava_prof_read waits for the stream and returns one kernel's launches and total milliseconds since
 * the clock was switched on; ava_prof_names lists the kernels seen, one per line. */
int ava_prof_enable(ava_engine* e, int32_t on);
int ava_prof_read(ava_engine* e, const char* kernel, int64_t* launches, double* ms);
int ava_prof_names(ava_engine* e, char* out, int32_t cap);

/* Per-block intermediates of the last step (row-major [rows, width] f32 copied to host), for teacher-forced parity
 * checks — the side-band of `Model::step_trace` (src/model/fstep/arch.rs:420-450).  Names: "h_lif", "spikes",
 * "x_lif", "h_mem", "qkveg", "y_raw", "y", "x_mem", "eng_qkv", "eng_o", "u", "a", "x_out".  Call ava_debug_keep(e, 1)
 * before the step; widths via ava_debug_width. */
int ava_debug_keep(ava_engine* e, int32_t on);
int64_t ava_debug_width(const ava_engine* e, const char* name);
int ava_debug_get(ava_engine* e, const char* name, int32_t block, float* out);

/* ---- checkpoints: the loader either side of the engine (src/ckpt.rs, src/arch.rs `Arch::from_flags`) --------------- */

typedef struct ava_ckpt ava_ckpt;

/* Text of the last loader error on this thread (never NULL). */
const char* ava_loader_error(void);
/* `ckpt::read` (src/ckpt.rs:16-18): opens a .safetensors file and checks its header (names, dtypes F32 / F16 / BF16,
 * shapes of at most 4 dimensions, data offsets that match).  The file is read into host memory once. */
int ava_ckpt_open(const char* path, ava_ckpt** out);
void ava_ckpt_close(ava_ckpt* c);
int32_t ava_ckpt_count(const ava_ckpt* c);
/* index of the tensor called `name`, or -1 */
int32_t ava_ckpt_find(const ava_ckpt* c, const char* name);
/* name, dtype text, rank and dims (4 slots, unused ones 1) of tensor i; any out pointer may be NULL */
int ava_ckpt_tensor(const ava_ckpt* c, int32_t i, const char** name, const char** dtype, int32_t* rank, int64_t* dims);
/* tensor i as f32 (n = its element count); integer tensors (U32: the counters of a state file) through read_u32 */
int ava_ckpt_read_f32(const ava_ckpt* c, int32_t i, float* out, int64_t n);
int ava_ckpt_read_u32(const ava_ckpt* c, int32_t i, uint32_t* out, int64_t n);
/* `Arch::from_flags` (src/arch.rs:273-420,596-607) on top of `cfg`: the one-line block options of an arch.txt.  Options
 * that only shape training or initial values are accepted and ignored; an option that adds a part the engine does not
 * have gives AVA_NOT_APPLICABLE with its name in ava_loader_error (the `fused_blocker` convention). */
int ava_arch_flags(const char* flags, ava_config* cfg);
/* `ckpt::detect` + `Config::with_arch` (src/ckpt.rs:21-60): the configuration a file was saved with.  vocab and d from
 * tok_emb, the block count from the highest b{i}, the engram's block from b{i}.eng.wq, the wide layer from b0.mlp.w1,
 * per-neuron thresholds from b{i}.mem.theta; `kind` ("S" or "D") and the arch.txt line (NULL or "" for none) are not
 * in the file and are given, as in the reference. */
int ava_config_from_ckpt(const ava_ckpt* c, const char* kind, const char* arch_flags, ava_config* out);
/* `load_auto` + `Model::set_int8` (src/ckpt.rs:51-76, src/model.rs:949-991): every tensor of the file into the engine,
 * the matrices quantised per output column as they go; call ava_engine_finalize afterwards. */
int ava_engine_load_ckpt(ava_engine* e, const ava_ckpt* c);

/* ---- carried state on disk (`State::save` / `State::load`, src/state.rs:1114-1329) ------------------------------- */

/* `Model::fingerprint` (src/state.rs:1075-1091) for the engine's model: FNV-1a over the configuration, every 97th value
 * of tok_emb, final.norm, and every 101st int8 weight of each block's w2 with its scales.  NOT the reference's value
 * (that one hashes the Debug text of its Rust Config and the f32 w2), so a state file is tied to this engine's model. */
uint64_t ava_engine_fingerprint(const ava_engine* e);
/* the engine a state belongs to */
ava_engine* ava_state_engine(const ava_state* s);
/* tokens read so far of a row (`State::seen`), set when a state is rebuilt from a file */
int ava_state_set_seen(ava_state* s, int32_t row, int64_t seen);
/* `State::save`: the state as a safetensors file under the reference's tensor names and shapes (meta.seen, meta.model,
 * meta.blocks, meta.cap, meta.hist, meta.hist_len, lif.{i}.{v,s,a} [rows, d], mem.{i}.{f,s} [rows * heads, hs, hs],
 * eng.{k,v} [rows, heads, S, hs] left-padded with eng.valid and eng.pad), written through PATH.tmp and a rename.
 * meta.hist is written empty: the token history feeds the reference's glance and magnitude codes, which the engine
 * does not have. */
int ava_state_save(const ava_state* s, const char* path);
/* `State::load`: a state that ava_state_save wrote for this engine's model (AVA_ERR_STATE when the file is not one, or
 * its fingerprint, block count or cap differ).  max_ctx: the engram ring's length, at least the stored length. */
int ava_state_load(ava_engine* e, const char* path, int32_t max_ctx, ava_state** out);
/* `ConvStore` (src/state.rs:1334-1384): one saved state per conversation in a folder.  The file of conversation `id` is
 * DIR/state-ID.safetensors when the id is short and plain (at most 64 letters, digits, '-' and '_'), else
 * DIR/state-hXXXXXXXXXXXXXXXX.safetensors with the FNV-1a hash of the id. */
int ava_conv_path(const char* dir, const char* id, char* out, int64_t n);
int ava_conv_save(const char* dir, const char* id, const ava_state* s);
/* `ConvStore::load`: *found = AVA_CONV_FRESH (no file; *out NULL), AVA_CONV_RESUMED (*out is the state) or
 * AVA_CONV_STALE (a file of another model, or unreadable: start fresh; *out NULL). */
#define AVA_CONV_FRESH 0
#define AVA_CONV_RESUMED 1
#define AVA_CONV_STALE 2
int ava_conv_load(ava_engine* e, const char* dir, const char* id, int32_t max_ctx, ava_state** out, int32_t* found);

/* ---- the step's callers: sampler and batched generation (src/diary.rs:686-744, src/state.rs:1388-1458) ----------- */

/* The configuration the engine was created with (valid while the engine lives). */
const ava_config* ava_engine_config(const ava_engine* e);
/* The CUDA device the engine runs on. */
int ava_engine_device(const ava_engine* e);
/* `SplitMix64::next_u64` (nn/data/src/rng.rs:24-28): advances *state and returns the next 64 bits. */
uint64_t ava_splitmix64_next(uint64_t* state);
/* `diary::pick` / `pick_traced` (src/diary.rs:686-744) on one row of host logits: the most likely token (lowest index
 * among equals) when temperature <= 0, else softmax(logits / temperature) in f32, the top_k most likely kept (ties in
 * index order), one draw of *rng_state over their mass.  logp (may be NULL): ln p(token) under the model at
 * temperature 1; sample_logp (may be NULL): ln p(token) under the sampler, 0 for a greedy pick. */
int ava_pick(const float* logits, int32_t vocab, float temperature, int32_t top_k, uint64_t* rng_state, uint32_t* token, float* logp,
             float* sample_logp);
/* One step with the next token of every row drawn on the device: `diary::pick` with the row's uniform number
 * uniform[r] in [0, 1) (what `(next_u64 >> 11) / 2^53` gives), the same token ava_pick draws from the same logits and
 * number.  No logits leave the device.  temperature <= 0: the greedy step.  AVA_NOT_APPLICABLE when top_k is above
 * 1024 (and below the vocabulary) or the vocabulary does not fit the sampler's shared memory (about 50,000). */
int ava_step_sample(ava_engine* e, ava_state* s, const uint32_t* tok, float temperature, int32_t top_k, const double* uniform, uint32_t* next);
/* The reference's `pick` and `stop` closures: the token for prompt `prompt_index` given its logits; whether the row
 * stops after the tokens written so far. */
typedef uint32_t (*ava_pick_fn)(void* user, int32_t prompt_index, const float* logits, int32_t vocab);
typedef int (*ava_stop_fn)(void* user, int32_t prompt_index, const uint32_t* tokens, int32_t n);
/* `state::generate` (src/state.rs:1388-1458): continuations of every prompt with carried state.  prompts: the ids of
 * all prompts one after another, prompt_len [n_prompts] (none empty).  The prompts are read in groups of at most
 * batch_rows rows, rows of one length in one chunked pass; then the group steps together, one token per pass, and a
 * row leaves at `eos` (not written), when `stop` says so, or after max_new tokens.  pick NULL: greedy, taken on the
 * device (no logits leave it); stop may be NULL.  max_ctx <= 0: longest prompt + max_new + 1 (the engram ring's
 * length).  out [n_prompts][max_new], out_len [n_prompts]. */
int ava_generate(ava_engine* e, const uint32_t* prompts, const int32_t* prompt_len, int32_t n_prompts, int32_t max_new, int32_t batch_rows,
                 int32_t max_ctx, uint32_t eos, ava_pick_fn pick, ava_stop_fn stop, void* user, uint32_t* out, int32_t* out_len);
/* The same loop with `diary::pick(logits, temperature, top_k, rng)` as the pick, one generator for all rows stepped in
 * the order the reference's loop calls it (the live rows of a group in order, every step): the tokens are those of
 * ava_generate with such a callback, but after the prompt the draws are taken on the device (ava_step_sample). */
int ava_generate_sampled(ava_engine* e, const uint32_t* prompts, const int32_t* prompt_len, int32_t n_prompts, int32_t max_new, int32_t batch_rows,
                         int32_t max_ctx, uint32_t eos, float temperature, int32_t top_k, uint64_t* rng_state, ava_stop_fn stop, void* user,
                         uint32_t* out, int32_t* out_len);

/* ---- single operators on host buffers (the S1 operator seam and the per-op kernels, for parity tests) ---------- */

/* `QW::matmul_rows` (src/int8.rs:124): y [m, dout] = x [m, din] . W.  Same bits as the reference's ordered sum. */
int ava_op_q8_matmul(int device, const float* x, int32_t m, const int8_t* q, const float* scale, int32_t din, int32_t dout, float* y);
/* The same through the event-sum kernel (E2, src/int8.rs:10-13,142-163): only the non-zero inputs of each row are
 * summed, in order; the same bits as the dense sum for any input. */
int ava_op_q8_event_matmul(int device, const float* x, int32_t m, const int8_t* q, const float* scale, int32_t din, int32_t dout, float* y);
/* The same product on the tensor cores (no counterpart in the reference): every product exact (three bf16 limbs of
 * each activation, the int8 weight exact in bf16), the f32 sum in the tensor core's order, so y agrees with
 * ava_op_q8_matmul to about 1e-6 of the sum of magnitudes, not bit for bit.  din % 64 == 0, dout % 4 == 0, else
 * AVA_NOT_APPLICABLE.  reps > 0 and ms_per_launch != NULL: also times reps launches of the product kernel. */
int ava_op_q8_tc_matmul(int device, const float* x, int32_t m, const int8_t* q, const float* scale, int32_t din, int32_t dout, float* y,
                        int32_t reps, float* ms_per_launch);
/* The device sampler alone (the kernel behind ava_step_sample) on m rows of host logits: next[r] is the token ava_pick
 * draws from logits[r] with the uniform number uniform[r].  temperature > 0. */
int ava_op_sample(int device, const float* logits, int32_t m, int32_t vocab, float temperature, int32_t top_k, const double* uniform, uint32_t* next);
/* `fstep::rmsnorm` (src/model/fstep.rs:207-220) on m rows of n. */
int ava_op_rmsnorm(int device, const float* x, const float* gain, int32_t m, int32_t n, float* y);
/* `fstep::arch::lif` (src/model/fstep/arch.rs:173-228) on m rows of d; theta/rho/gain/a0/a1 may be NULL. */
int ava_op_lif(int device, const float* cur, const float* beta, const float* theta, const float* rho, const float* gain,
               int32_t spikes, const float* v0, const float* s0, const float* a0, int32_t m, int32_t d, float* s1, float* v1,
               float* a1);
/* kth_largest + mask + relu(^2) (src/model/fstep.rs:295-299, src/model/fstep/arch.rs:982-989) on m rows of n. */
int ava_op_kwta(int device, const float* u, int32_t m, int32_t n, int32_t k, int32_t relu2, float* a);
/* `head_rows` without momentum (src/model/fstep/arch.rs:256-337) for m independent heads of size hs:
 * e, v, w, ah, qg, ex [m, hs]; qw, qa [m]; f [m, hs, hs] updated in place; y [m, hs]. */
int ava_op_mem_heads(int device, int32_t m, int32_t hs, const float* e, const float* v, const float* w, const float* ah,
                     const float* qg, const float* ex, const float* qw, const float* qa, float* f, float* y);
/* The same product for rows of small integers (spikes in {-2..2}) on the tensor cores, added to y: y += (x . q) * scale
 * (no counterpart in the reference).  One bf16 limb each side is exact for such operands, and every partial sum is an
 * integer below 2^24, so the f32 accumulator is exact whatever its order: the result is the ordered sum's bits
 * (src/int8.rs:315-331).  m % 128, din % 64, dout % 4, else AVA_NOT_APPLICABLE. */
int ava_op_q8_spike_tc_matmul(int device, const float* x, int32_t m, const int8_t* q, const float* scale, int32_t din, int32_t dout, float* y);
/* No counterpart in the reference.  ava_op_mem_heads for callers that cannot allocate device memory (a latency-critical
 * thread that must not take the allocator's device-wide lock, a process whose GPU memory was handed out in full at
 * start-up): every pointer is DEVICE memory, `stream` is a cudaStream_t (NULL: the default stream), f [m, hs, hs] is
 * updated in place and y [m, hs] written.  e, v, w, ah, qg and ex must be 16-byte aligned (the kernel reads them with
 * bulk copies; a sub-view of a larger buffer must keep that alignment), qw, qa, f and y 4-byte aligned: anything else
 * is refused with AVA_ERR_ARG before a launch.  The kernel's scratch is a built-in device array of
 * AVA_STATIC_SCRATCH_BYTES that every GPU loading the library holds until exit; m * hs * hs above
 * AVA_STATIC_SCRATCH_FLOATS is refused with AVA_ERR_CAPACITY (text from ava_static_last_error).  All calls on a device
 * share that array: calls that overlap on the GPU race.  The first call on a device looks the array's address up; make
 * it before any stream capture.  The call makes `device` the calling thread's current device and returns after the
 * stream has drained. */
#define AVA_STATIC_SCRATCH_FLOATS 4194304
#define AVA_STATIC_SCRATCH_BYTES (4 * AVA_STATIC_SCRATCH_FLOATS)
int ava_mem_heads_static(int device, void* stream, int32_t m, int32_t hs, const float* e, const float* v, const float* w, const float* ah,
                         const float* qg, const float* ex, const float* qw, const float* qa, float* f, float* y);
const char* ava_static_last_error(void);
/* `attend` (src/model/fstep.rs:303-327) for m heads over n keys/values of hs (f32, or rounded to bf16 first). */
int ava_op_attend(int device, int32_t m, int32_t n, int32_t hs, int32_t bf16_store, const float* q, const float* kc,
                  const float* vc, float* out);

/* No counterpart in the reference (it reads the engram once per token, src/model/fstep.rs:303-356).  The causal read of
 * a whole chunk on the tensor cores, alone, on host buffers: `rows` stores of head size 64 kept in bf16, each holding n0
 * tokens (k_prev, v_prev [rows][d / 64][n0][64]) from ring slot `start` on; t tokens with qkv [t][rows][3 d] join them and
 * o [t][rows][d] gets each token's softmax(K q / 8) V over the keys up to and including its own.  Agrees with the
 * one-token read to rounding.  d % 64 != 0: AVA_NOT_APPLICABLE. */
int ava_op_engram_chunk(int device, int32_t rows, int32_t t, int32_t n0, int32_t start, int32_t d, const float* qkv, const float* k_prev,
                        const float* v_prev, float* o);
/* No counterpart in the reference (its chunked memory multiplies with its tensor library's matmul,
 * src/arch.rs:1243-1327).  The batched limb product of the chunked memory alone, on host buffers: c[b] = a[b] . b[b]^T
 * (a [batch][m][k], b [batch][n][k], c [batch][m][n]); with colscale [batch][n], c = colscale[b][n] * c + a . b^T and
 * c_limb_sum (may be NULL) gets the exact sum of the three bf16 limbs written for the new c.  m % 128, k % 64, n % 4,
 * else AVA_NOT_APPLICABLE. */
int ava_op_tc_bgemm(int device, int32_t batch, int32_t m, int32_t n, int32_t k, const float* a, const float* b, const float* colscale, float* c,
                    float* c_limb_sum);
/* The chunk-parallel form of the fast-weight memory alone, on host buffers: `delta_chunk` / `chunk_core`
 * (src/arch.rs:1151-1173, 1243-1327) with per-channel gates and no momentum, the big products on the tensor cores.
 * Like the reference's it agrees with the token loop to rounding (1e-4 of max(1, max|ref|), src/arch/tests.rs:700-753),
 * not bit for bit.  t tokens (a multiple of 64) of hb head-rows of size hs (a multiple of 128, else
 * AVA_NOT_APPLICABLE), inputs [t][hb][hs]: qn unit query, e unit erase direction, w write key, ah erase key, v value,
 * la log rate (<= 0).  f [hb][hs key][hs value] is advanced in place, y [t][hb][hs] gets the reads.  When a chunk's
 * log rates sum below -60 the form is out of its range: *out_of_range = 1, f and y untouched, AVA_OK. */
int ava_op_mem_chunk(int device, int32_t t, int32_t hb, int32_t hs, const float* qn, const float* e, const float* w, const float* ah, const float* v,
                     const float* la, float* f, float* y, int32_t* out_of_range);
/* Testing aid for the kernels' bounded waits; no counterpart in the reference (its waits are host-side joins).  Runs
 * the fast-weight kernel on m pattern-filled heads of size hs with the byte count of row chunk `chunk` over-stated by
 * 16 on every block's first item and a poll limit of `poll_limit`, so that wait runs out without any copy failing.
 * Returns AVA_ERR_CUDA when the kernel flagged the time-out (what a step would return), AVA_OK when it did not;
 * *state_changed = 1 if any bit of the state in device memory changed (a block that gave up must store nothing). */
int ava_debug_mem_heads_wait_runs_out(int device, int32_t m, int32_t hs, int32_t chunk, uint32_t poll_limit, int32_t* state_changed);

/* The engine's exp / ln / x^-1/2, evaluated on the host with the operation sequence the kernels use (same bits). */
float ava_host_expf(float x);
float ava_host_logf(float x);
float ava_host_rsqrtf(float x);
float ava_host_sinf(float x);
float ava_host_cosf(float x);
/* The same evaluated on the device, n values (tests that host and device agree bit for bit). which: 0 exp, 1 ln, 2 x^-1/2. */
int ava_op_math(int device, int32_t which, const float* x, int64_t n, float* y);

#ifdef __cplusplus
}
#endif
#endif
