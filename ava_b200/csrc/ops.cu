// Single operators of the block step on host buffers: the kernels behind the step, callable one at a time so that a
// parity test can feed an operator exactly the inputs the reference's code would see (teacher forcing).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <vector>

#include "../../include/ava_engine.h"
#include "ava_math.h"
#include "kernels.cuh"

namespace {

using namespace ava;

struct Tmp {
    void* p = nullptr;
    ~Tmp() {
        if (p) cudaFree(p);
    }
    template <typename T>
    T* as() { return reinterpret_cast<T*>(p); }
};

#define OCK(call)                                   \
    do {                                            \
        if ((call) != cudaSuccess) return AVA_ERR_CUDA; \
    } while (0)

cudaError_t up(Tmp& t, const void* src, size_t bytes) {
    cudaError_t e = cudaMalloc(&t.p, bytes ? bytes : 1);
    if (e != cudaSuccess) return e;
    return src && bytes ? cudaMemcpy(t.p, src, bytes, cudaMemcpyHostToDevice) : cudaSuccess;
}

int begin(int device) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return AVA_ERR_CUDA;
    take_launch_error();  // what an earlier, failed call left
    return cudaSetDevice(device) == cudaSuccess ? AVA_OK : AVA_ERR_CUDA;
}

int end_() {
    if (take_launch_error() != cudaSuccess) return AVA_ERR_CUDA;
    if (cudaGetLastError() != cudaSuccess) return AVA_ERR_CUDA;
    return cudaDeviceSynchronize() == cudaSuccess ? AVA_OK : AVA_ERR_CUDA;
}

}  // namespace

extern "C" {

static int q8_matmul_impl(int device, const float* x, int32_t m, const int8_t* q, const float* scale, int32_t din, int32_t dout, float* y, bool event);

int ava_op_q8_matmul(int device, const float* x, int32_t m, const int8_t* q, const float* scale, int32_t din, int32_t dout, float* y) {
    return q8_matmul_impl(device, x, m, q, scale, din, dout, y, false);
}
int ava_op_q8_event_matmul(int device, const float* x, int32_t m, const int8_t* q, const float* scale, int32_t din, int32_t dout, float* y) {
    return q8_matmul_impl(device, x, m, q, scale, din, dout, y, true);
}

static int q8_matmul_impl(int device, const float* x, int32_t m, const int8_t* q, const float* scale, int32_t din, int32_t dout, float* y, bool event) {
    if (!x || !q || !scale || !y || m <= 0 || din <= 0 || dout <= 0) return AVA_ERR_ARG;
    if (din % 16 || dout % 4) return AVA_NOT_APPLICABLE;
    int rc = begin(device);
    if (rc) return rc;
    Tmp dx, dq, ds, dy;
    OCK(up(dx, x, (size_t)m * din * 4));
    OCK(up(dq, q, (size_t)din * dout));
    OCK(up(ds, scale, (size_t)dout * 4));
    OCK(up(dy, nullptr, (size_t)m * dout * 4));
    GemmArgs g{};
    g.A = dx.as<float>(); g.lda = din; g.W = dq.as<int8_t>(); g.ldw = dout; g.scale = ds.as<float>();
    g.C = dy.as<float>(); g.ldc = dout; g.M = m; g.N = dout; g.K = din;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    // the kernels a step of this many rows would take (the engine's own choice: see `gemm` in engine.cu)
    if (event) {
        if (!launch_q8_event(0, g, EPI_STORE)) return AVA_NOT_APPLICABLE;
    } else if (!(m > 16 && launch_q8_gemm2(0, g, EPI_STORE, sms))) {
        launch_q8_gemm(0, g, EPI_STORE, sms);
    }
    if ((rc = end_())) return rc;
    OCK(cudaMemcpy(y, dy.p, (size_t)m * dout * 4, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

int ava_op_q8_tc_matmul(int device, const float* x, int32_t m, const int8_t* q, const float* scale, int32_t din, int32_t dout, float* y,
                        int32_t reps, float* ms_per_launch) {
    if (!x || !q || !scale || !y || m <= 0 || din <= 0 || dout <= 0 || reps < 0) return AVA_ERR_ARG;
    if (din % 64 || dout % 4) return AVA_NOT_APPLICABLE;
    int rc = begin(device);
    if (rc) return rc;
    Tmp dx, dq, ds, dy, dl, dw, dst;
    OCK(up(dx, x, (size_t)m * din * 4));
    OCK(up(dq, q, (size_t)din * dout));
    OCK(up(ds, scale, (size_t)dout * 4));
    OCK(up(dy, nullptr, (size_t)m * dout * 4));
    OCK(up(dl, nullptr, (size_t)3 * m * din * 2));
    OCK(up(dw, nullptr, (size_t)din * dout * 2));
    OCK(up(dst, nullptr, 4));
    OCK(cudaMemset(dst.p, 0, 4));
    launch_widen_transpose(0, dq.as<int8_t>(), din, dout, dw.as<uint16_t>());
    launch_split3(0, dx.as<float>(), (int64_t)m * din, dl.as<uint16_t>());
    TcGemmArgs g{};
    g.a_limbs = dl.as<uint16_t>(); g.w_bf16 = dw.as<uint16_t>(); g.scale = ds.as<float>();
    g.C = dy.as<float>(); g.ldc = dout; g.M = m; g.N = dout; g.K = din; g.status = dst.as<uint32_t>();
    if (!launch_tc_gemm(0, g, EPI_STORE)) return AVA_NOT_APPLICABLE;
    if ((rc = end_())) return rc;
    uint32_t st = 0;
    OCK(cudaMemcpy(&st, dst.p, 4, cudaMemcpyDeviceToHost));
    if (st) return AVA_ERR_STATE;
    OCK(cudaMemcpy(y, dy.p, (size_t)m * dout * 4, cudaMemcpyDeviceToHost));
    if (reps > 0 && ms_per_launch) {  // the product alone, inputs resident, back to back
        cudaEvent_t e0, e1;
        OCK(cudaEventCreate(&e0));
        OCK(cudaEventCreate(&e1));
        OCK(cudaEventRecord(e0, 0));
        for (int i = 0; i < reps; ++i) launch_tc_gemm(0, g, EPI_STORE);
        OCK(cudaEventRecord(e1, 0));
        if ((rc = end_())) return rc;
        float ms = 0.0f;
        OCK(cudaEventElapsedTime(&ms, e0, e1));
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        *ms_per_launch = ms / (float)reps;
    }
    return AVA_OK;
}

/* Rows of small integers (spikes) times int8 weights on the tensor cores, added to y: y += (x . q) * scale.  Every product
 * and partial sum is an integer below 2^24, so the result is the ordered sum's bits (checked against the event sum). */
int ava_op_q8_spike_tc_matmul(int device, const float* x, int32_t m, const int8_t* q, const float* scale, int32_t din, int32_t dout, float* y) {
    if (!x || !q || !scale || !y || m <= 0 || din <= 0 || dout <= 0) return AVA_ERR_ARG;
    if (din % 64 || dout % 4 || m % 128) return AVA_NOT_APPLICABLE;
    int rc = begin(device);
    if (rc) return rc;
    Tmp dx, dq, ds, dy, dl, dw, dst;
    OCK(up(dx, x, (size_t)m * din * 4));
    OCK(up(dq, q, (size_t)din * dout));
    OCK(up(ds, scale, (size_t)dout * 4));
    OCK(up(dy, y, (size_t)m * dout * 4));
    OCK(up(dl, nullptr, (size_t)m * din * 2));
    OCK(up(dw, nullptr, (size_t)din * dout * 2));
    OCK(up(dst, nullptr, 4));
    OCK(cudaMemset(dst.p, 0, 4));
    launch_widen_transpose(0, dq.as<int8_t>(), din, dout, dw.as<uint16_t>());
    launch_round_bf16(0, dx.as<float>(), (int64_t)m * din, dl.as<uint16_t>());
    TcbArgs t{};
    t.a = dl.as<uint16_t>(); t.rows_a = m; t.b = dw.as<uint16_t>(); t.rows_b = dout;
    t.C = dy.as<float>(); t.ldc = dout; t.M = m; t.N = dout; t.K = din; t.batch = 1; t.colscale = ds.as<float>(); t.status = dst.as<uint32_t>();
    if (!launch_tc_bgemm(0, t, TCB_SCALE_ADD)) return AVA_NOT_APPLICABLE;
    if ((rc = end_())) return rc;
    uint32_t st = 0;
    OCK(cudaMemcpy(&st, dst.p, 4, cudaMemcpyDeviceToHost));
    if (st) return AVA_ERR_STATE;
    OCK(cudaMemcpy(y, dy.p, (size_t)m * dout * 4, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

int ava_op_sample(int device, const float* logits, int32_t m, int32_t vocab, float temperature, int32_t top_k, const double* uniform, uint32_t* next) {
    if (!logits || !uniform || !next || m <= 0 || vocab <= 0) return AVA_ERR_ARG;
    int rc = begin(device);
    if (rc) return rc;
    Tmp dl, du, dn;
    OCK(up(dl, logits, (size_t)m * vocab * 4));
    OCK(up(du, uniform, (size_t)m * 8));
    OCK(up(dn, nullptr, (size_t)m * 4));
    if (!launch_sample(0, dl.as<float>(), m, vocab, temperature, top_k, du.as<double>(), dn.as<uint32_t>())) return AVA_NOT_APPLICABLE;
    if ((rc = end_())) return rc;
    OCK(cudaMemcpy(next, dn.p, (size_t)m * 4, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

int ava_op_rmsnorm(int device, const float* x, const float* gain, int32_t m, int32_t n, float* y) {
    if (!x || !gain || !y || m <= 0 || n <= 0) return AVA_ERR_ARG;
    int rc = begin(device);
    if (rc) return rc;
    Tmp dx, dg, dy;
    OCK(up(dx, x, (size_t)m * n * 4));
    OCK(up(dg, gain, (size_t)n * 4));
    OCK(up(dy, nullptr, (size_t)m * n * 4));
    launch_rmsnorm(0, dx.as<float>(), dg.as<float>(), m, n, dy.as<float>());
    if ((rc = end_())) return rc;
    OCK(cudaMemcpy(y, dy.p, (size_t)m * n * 4, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

int ava_op_lif(int device, const float* cur, const float* beta, const float* theta, const float* rho, const float* gain, int32_t spikes,
               const float* v0, const float* s0, const float* a0, int32_t m, int32_t d, float* s1, float* v1, float* a1) {
    if (!cur || !beta || !v0 || !s0 || !s1 || !v1 || m <= 0 || d <= 0) return AVA_ERR_ARG;
    const bool alif = rho && gain;
    if (alif && (!a0 || !a1)) return AVA_ERR_ARG;
    int rc = begin(device);
    if (rc) return rc;
    const size_t md = (size_t)m * d * 4, dd = (size_t)d * 4;
    Tmp dc, db, dt, dr, dg, dv, ds, da;
    OCK(up(dc, cur, md));
    OCK(up(db, beta, dd));
    if (theta) OCK(up(dt, theta, dd));
    if (alif) {
        OCK(up(dr, rho, dd));
        OCK(up(dg, gain, dd));
        OCK(up(da, a0, md));
    }
    OCK(up(dv, v0, md));
    OCK(up(ds, s0, md));
    LifParams p{};
    p.beta = db.as<float>(); p.theta = theta ? dt.as<float>() : nullptr; p.rho = alif ? dr.as<float>() : nullptr;
    p.gain = alif ? dg.as<float>() : nullptr; p.v = dv.as<float>(); p.s = ds.as<float>(); p.a = alif ? da.as<float>() : nullptr;
    p.spikes = spikes; p.lif_scale = 0;
    launch_lif(0, dc.as<float>(), p, m, d);
    if ((rc = end_())) return rc;
    OCK(cudaMemcpy(s1, ds.p, md, cudaMemcpyDeviceToHost));
    OCK(cudaMemcpy(v1, dv.p, md, cudaMemcpyDeviceToHost));
    if (alif) OCK(cudaMemcpy(a1, da.p, md, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

int ava_op_kwta(int device, const float* u, int32_t m, int32_t n, int32_t k, int32_t relu2, float* a) {
    if (!u || !a || m <= 0 || n <= 0 || k <= 0) return AVA_ERR_ARG;
    int rc = begin(device);
    if (rc) return rc;
    Tmp du, da;
    OCK(up(du, u, (size_t)m * n * 4));
    OCK(up(da, nullptr, (size_t)m * n * 4));
    launch_kwta(0, du.as<float>(), m, n, k, relu2, da.as<float>());
    if ((rc = end_())) return rc;
    OCK(cudaMemcpy(a, da.p, (size_t)m * n * 4, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

int ava_op_mem_heads(int device, int32_t m, int32_t hs, const float* e, const float* v, const float* w, const float* ah, const float* qg,
                     const float* ex, const float* qw, const float* qa, float* f, float* y) {
    if (!e || !v || !w || !ah || !qg || !ex || !qw || !qa || !f || !y || m <= 0 || hs <= 0) return AVA_ERR_ARG;
    int cw, rb;
    if (hs % 16 || !mem_heads_tiling(hs, &cw, &rb)) return AVA_NOT_APPLICABLE;
    int rc = begin(device);
    if (rc) return rc;
    const size_t vb = (size_t)m * hs * 4, fb = (size_t)m * hs * hs * 4;
    Tmp de, dv, dw, dah, dqg, dex, dqw, dqa, df, dy, dst;
    OCK(up(de, e, vb)); OCK(up(dv, v, vb)); OCK(up(dw, w, vb)); OCK(up(dah, ah, vb)); OCK(up(dqg, qg, vb)); OCK(up(dex, ex, vb));
    OCK(up(dqw, qw, (size_t)m * 4)); OCK(up(dqa, qa, (size_t)m * 4));
    OCK(up(df, f, fb));
    OCK(up(dy, nullptr, vb));
    OCK(up(dst, nullptr, 4));
    OCK(cudaMemset(dst.p, 0, 4));
    Tmp dft, drr;  // the slice-major copy the kernels work on; the token's rr
    OCK(up(dft, nullptr, fb));
    OCK(up(drr, nullptr, vb));
    launch_retile(0, df.as<float>(), dft.as<float>(), m, hs, cw, 1);
    // what a decode step runs: the streaming pass (here with no update pending), which leaves the token's own update
    // pending, then that update applied alone, as every reader of the state other than the next pass would first do
    MemStreamArgs a{};
    a.f = dft.as<float>(); a.M = m; a.nh = 1; a.hs = hs; a.cw = cw;
    a.e = de.as<float>(); a.qg = dqg.as<float>(); a.v = dv.as<float>(); a.qw = dqw.as<float>(); a.qa = dqa.as<float>();
    a.y = dy.as<float>(); a.rr_out = drr.as<float>();
    if (!launch_mem_stream(0, a)) return AVA_NOT_APPLICABLE;
    launch_mem_flush(0, dft.as<float>(), dex.as<float>(), dw.as<float>(), dah.as<float>(), dv.as<float>(), drr.as<float>(), m, hs, cw);
    launch_retile(0, dft.as<float>(), df.as<float>(), m, hs, cw, 0);
    if ((rc = end_())) return rc;
    uint32_t st = 0;
    OCK(cudaMemcpy(&st, dst.p, 4, cudaMemcpyDeviceToHost));
    if (st) return AVA_ERR_CUDA;
    OCK(cudaMemcpy(f, df.p, fb, cudaMemcpyDeviceToHost));
    OCK(cudaMemcpy(y, dy.p, vb, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

/* The batched limb product of the chunked memory alone: C[b] = A[b] . B[b]^T (+ colscale[b][n] * C_in when colscale is
 * given), A [batch][M][K], B [batch][N][K], C [batch][M][N] f32 on the host; limbs [3][batch * M][N] of the result are
 * returned as their exact sum in c_limb_sum when it is not NULL (TCB_DECAY only). */
int ava_op_tc_bgemm(int device, int32_t batch, int32_t m, int32_t n, int32_t k, const float* a, const float* b, const float* colscale, float* c,
                    float* c_limb_sum) {
    if (!a || !b || !c || batch <= 0 || m <= 0 || n <= 0 || k <= 0) return AVA_ERR_ARG;
    if (m % 128 || k % 64 || n % 4) return AVA_NOT_APPLICABLE;
    int rc = begin(device);
    if (rc) return rc;
    const size_t na = (size_t)batch * m * k, nb = (size_t)batch * n * k, nc = (size_t)batch * m * n;
    Tmp da, db, dc, dla, dlb, dcs, dcl, dst;
    OCK(up(da, a, na * 4)); OCK(up(db, b, nb * 4)); OCK(up(dc, c, nc * 4));
    OCK(up(dla, nullptr, na * 6)); OCK(up(dlb, nullptr, nb * 6)); OCK(up(dst, nullptr, 4));
    OCK(cudaMemset(dst.p, 0, 4));
    launch_split3(0, da.as<float>(), (int64_t)na, dla.as<uint16_t>());
    launch_split3(0, db.as<float>(), (int64_t)nb, dlb.as<uint16_t>());
    TcbArgs t{};
    t.a = dla.as<uint16_t>(); t.b = dlb.as<uint16_t>(); t.rows_a = (int64_t)batch * m; t.rows_b = (int64_t)batch * n;
    t.C = dc.as<float>(); t.ldc = n; t.c_batch_stride = (int64_t)m * n; t.M = m; t.N = n; t.K = k; t.batch = batch; t.status = dst.as<uint32_t>();
    if (colscale) {
        OCK(up(dcs, colscale, (size_t)batch * n * 4));
        OCK(up(dcl, nullptr, nc * 6));
        t.colscale = dcs.as<float>(); t.colscale_batch_stride = n; t.c_limbs = dcl.as<uint16_t>(); t.c_limb_plane = (int64_t)nc;
    }
    if (!launch_tc_bgemm(0, t, colscale ? TCB_DECAY : TCB_STORE)) return AVA_NOT_APPLICABLE;
    if ((rc = end_())) return rc;
    uint32_t st = 0;
    OCK(cudaMemcpy(&st, dst.p, 4, cudaMemcpyDeviceToHost));
    if (st) return AVA_ERR_CUDA;
    OCK(cudaMemcpy(c, dc.p, nc * 4, cudaMemcpyDeviceToHost));
    if (colscale && c_limb_sum) {
        std::vector<uint16_t> l(nc * 3);
        OCK(cudaMemcpy(l.data(), dcl.p, nc * 6, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < nc; ++i) c_limb_sum[i] = (bf16_to_f(l[i]) + bf16_to_f(l[nc + i])) + bf16_to_f(l[2 * nc + i]);
    }
    return AVA_OK;
}

/* The chunk-parallel form of the fast-weight memory alone (tensor-core products; agrees with the token loop to
 * rounding, not bit for bit).  t tokens (a multiple of 64) of hb head-rows of size hs (a multiple of 128), inputs
 * time-major [t][hb][hs]: unit query qn, unit erase direction e, write key w, erase key ah, value v, log rate la; the
 * state f [hb][hs(key)][hs(value)] is advanced in place, y [t][hb][hs] receives the reads.  *out_of_range is set to 1
 * (and nothing else is written) when a chunk's rates are too strong for this form; the caller then uses the token loop. */
int ava_op_mem_chunk(int device, int32_t t, int32_t hb, int32_t hs, const float* qn, const float* e, const float* w, const float* ah, const float* v,
                     const float* la, float* f, float* y, int32_t* out_of_range) {
    if (!qn || !e || !w || !ah || !v || !la || !f || !y || !out_of_range || t <= 0 || hb <= 0 || hs <= 0) return AVA_ERR_ARG;
    if (!mem_chunk_covers(hs, t, 0.0f)) return AVA_NOT_APPLICABLE;
    int rc = begin(device);
    if (rc) return rc;
    const size_t vn = (size_t)t * hb * hs, fn = (size_t)hb * hs * hs;
    Tmp dq, de, dw, da, dv, dl, df, dy, dws, dfl;
    OCK(up(dq, qn, vn * 4)); OCK(up(de, e, vn * 4)); OCK(up(dw, w, vn * 4)); OCK(up(da, ah, vn * 4)); OCK(up(dv, v, vn * 4)); OCK(up(dl, la, vn * 4));
    OCK(up(df, f, fn * 4)); OCK(up(dy, nullptr, vn * 4)); OCK(up(dfl, nullptr, 8));
    OCK(cudaMemset(dfl.p, 0, 8));
    ChunkArgs c{};
    c.HB = hb; c.hs = hs; c.nC = t / 64; c.cw = hs; c.tok_stride = (int64_t)hb * hs;
    c.qn = dq.as<float>(); c.e = de.as<float>(); c.w = dw.as<float>(); c.ah = da.as<float>(); c.v = dv.as<float>(); c.la = dl.as<float>();
    c.y = dy.as<float>(); c.F = df.as<float>(); c.flags = dfl.as<uint32_t>(); c.status = dfl.as<uint32_t>() + 1;
    OCK(up(dws, nullptr, mem_chunk_workspace_bytes(hb, hs, c.nC)));
    mem_chunk_carve(c, dws.p);
    if (!launch_mem_chunk_scale(0, c)) return AVA_NOT_APPLICABLE;
    uint32_t fl[2] = {0, 0};
    OCK(cudaMemcpy(fl, dfl.p, 8, cudaMemcpyDeviceToHost));
    *out_of_range = (int32_t)(fl[0] & 1u);
    if (*out_of_range) return end_();
    if (!launch_mem_chunk_rest(0, c)) return AVA_NOT_APPLICABLE;
    if ((rc = end_())) return rc;
    OCK(cudaMemcpy(fl, dfl.p, 8, cudaMemcpyDeviceToHost));
    if (fl[1]) return AVA_ERR_CUDA;
    OCK(cudaMemcpy(f, df.p, fn * 4, cudaMemcpyDeviceToHost));
    OCK(cudaMemcpy(y, dy.p, vn * 4, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

/* Testing aid for the kernels' bounded waits (no GPU fault involved: every copy completes, only a barrier is told to
 * expect 16 bytes more than will ever arrive).  Runs the fast-weight update + read on m heads of size hs whose state
 * is filled with a pattern, with chunk `chunk` of every block's first item mis-counted and a poll limit of
 * `poll_limit`, so the wait on that chunk runs out.  Returns what a step would return for the raised status word
 * (AVA_ERR_CUDA when the time-out was flagged, AVA_OK when it was not) and sets *state_changed to 1 when any bit of the
 * state in device memory differs from the pattern afterwards (it must not: a block that gave up stores nothing). */
int ava_debug_mem_heads_wait_runs_out(int device, int32_t m, int32_t hs, int32_t chunk, uint32_t poll_limit, int32_t* state_changed) {
    int cw, rb;
    if (!state_changed || m <= 0 || hs % 16 || !mem_heads_tiling(hs, &cw, &rb) || chunk < 0 || chunk >= hs / rb || poll_limit == 0) return AVA_ERR_ARG;
    int rc = begin(device);
    if (rc) return rc;
    const size_t vn = (size_t)m * hs, fn = (size_t)m * hs * hs;
    std::vector<float> hv(vn), hf(fn), back(fn);
    for (size_t i = 0; i < vn; ++i) hv[i] = 0.01f * (float)((i * 37) % 101) - 0.5f;
    for (size_t i = 0; i < fn; ++i) hf[i] = 0.001f * (float)((i * 131) % 1999) - 1.0f;
    Tmp dv, dq, df, dy, dst;
    OCK(up(dv, hv.data(), vn * 4)); OCK(up(dq, hv.data(), (size_t)m * 4)); OCK(up(df, hf.data(), fn * 4)); OCK(up(dy, nullptr, vn * 4)); OCK(up(dst, nullptr, 4));
    OCK(cudaMemset(dst.p, 0, 4));
    MemHeadsArgs a{};
    a.f = df.as<float>(); a.M = m; a.nh = 1; a.hs = hs; a.cw = cw; a.chunk_rows = rb;
    a.e = a.v = a.w = a.ah = a.qg = a.ex = dv.as<float>(); a.qw = a.qa = dq.as<float>(); a.y = dy.as<float>(); a.status = dst.as<uint32_t>();
    a.wait_limit = poll_limit;
    a.fault_chunk_plus1 = chunk + 1;
    launch_mem_heads_seq(0, a, 1);
    if ((rc = end_())) return rc;
    uint32_t st = 0;
    OCK(cudaMemcpy(&st, dst.p, 4, cudaMemcpyDeviceToHost));
    OCK(cudaMemcpy(back.data(), df.p, fn * 4, cudaMemcpyDeviceToHost));
    *state_changed = std::memcmp(back.data(), hf.data(), fn * 4) != 0;
    return (st & ST_WAIT_TIMEOUT) ? AVA_ERR_CUDA : AVA_OK;
}

/* The engram's causal read over a whole chunk on the tensor cores, alone (head size 64, bf16 store).  rows stores, each
 * holding n0 tokens already (k_prev, v_prev [rows][d / 64][n0][64], rounded to bf16 as the store keeps them) from ring
 * slot `start` on; then t tokens whose q | k | v are qkv [t][rows][3 d]: their keys and values join the store and
 * o [t][rows][d] gets every token's read over the keys up to and including its own. */
int ava_op_engram_chunk(int device, int32_t rows, int32_t t, int32_t n0, int32_t start, int32_t d, const float* qkv, const float* k_prev,
                        const float* v_prev, float* o) {
    if (!qkv || !o || rows <= 0 || t <= 0 || n0 < 0 || start < 0 || d <= 0 || (n0 > 0 && (!k_prev || !v_prev))) return AVA_ERR_ARG;
    if (d % 64) return AVA_NOT_APPLICABLE;
    int rc = begin(device);
    if (rc) return rc;
    const int nh = d / 64, cap = start + n0 + t + 5;  // a few slots never written: their bytes must not matter
    const size_t store = (size_t)rows * nh * cap * 64;
    std::vector<uint16_t> ks(store, 0x7fc0), vs(store, 0x7fc0);  // NaN patterns wherever nothing is stored
    for (int r = 0; r < rows; ++r)
        for (int hh = 0; hh < nh; ++hh)
            for (int j = 0; j < n0; ++j)
                for (int x = 0; x < 64; ++x) {
                    const size_t src = (((size_t)r * nh + hh) * n0 + j) * 64 + x, dst = (((size_t)r * nh + hh) * cap + start + j) * 64 + x;
                    ks[dst] = f_to_bf16(k_prev[src]);
                    vs[dst] = f_to_bf16(v_prev[src]);
                }
    std::vector<int32_t> hn(rows, n0), hs_(rows, start);
    Tmp dq, dk, dv, dn, dstart, dout, dst;
    OCK(up(dq, qkv, (size_t)t * rows * 3 * d * 4));
    OCK(up(dk, ks.data(), store * 2)); OCK(up(dv, vs.data(), store * 2));
    OCK(up(dn, hn.data(), rows * 4)); OCK(up(dstart, hs_.data(), rows * 4));
    OCK(up(dout, nullptr, (size_t)t * rows * d * 4)); OCK(up(dst, nullptr, 4));
    OCK(cudaMemset(dst.p, 0, 4));
    EngramChunkArgs a{};
    a.qkv = dq.as<float>(); a.o = dout.as<float>(); a.k = dk.p; a.v = dv.p; a.n = dn.as<int32_t>(); a.start = dstart.as<int32_t>();
    a.M = rows; a.d = d; a.hs = 64; a.cap = cap; a.T = t; a.bf16 = 1; a.status = dst.as<uint32_t>();
    if (!launch_engram_chunk(0, a)) return AVA_NOT_APPLICABLE;
    if ((rc = end_())) return rc;
    uint32_t st = 0;
    OCK(cudaMemcpy(&st, dst.p, 4, cudaMemcpyDeviceToHost));
    if (st) return AVA_ERR_CUDA;
    OCK(cudaMemcpy(hn.data(), dn.p, rows * 4, cudaMemcpyDeviceToHost));
    for (int r = 0; r < rows; ++r)
        if (hn[r] != n0 + t) return AVA_ERR_CUDA;
    OCK(cudaMemcpy(o, dout.p, (size_t)t * rows * d * 4, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

int ava_op_attend(int device, int32_t m, int32_t n, int32_t hs, int32_t bf16_store, const float* q, const float* kc, const float* vc, float* out) {
    if (!q || !kc || !vc || !out || m <= 0 || n <= 0 || hs <= 0) return AVA_ERR_ARG;
    int rc = begin(device);
    if (rc) return rc;
    // m heads as one row of width d = m * hs; the first n - 1 keys/values are laid in the store, the last one arrives
    // as this token's key and value
    const int d = m * hs;
    const size_t el = bf16_store ? 2 : 4;
    std::vector<float> qkv((size_t)3 * d);
    for (int hh = 0; hh < m; ++hh)
        for (int x = 0; x < hs; ++x) {
            qkv[hh * hs + x] = q[(size_t)hh * hs + x];
            qkv[d + hh * hs + x] = kc[((size_t)hh * n + (n - 1)) * hs + x];
            qkv[2 * d + hh * hs + x] = vc[((size_t)hh * n + (n - 1)) * hs + x];
        }
    std::vector<unsigned char> ks((size_t)d * n * el, 0), vs((size_t)d * n * el, 0);
    for (int hh = 0; hh < m; ++hh)
        for (int j = 0; j + 1 < n; ++j)
            for (int x = 0; x < hs; ++x) {
                const size_t i = ((size_t)hh * n + j) * hs + x;
                if (bf16_store) {
                    reinterpret_cast<uint16_t*>(ks.data())[i] = f_to_bf16(kc[i]);
                    reinterpret_cast<uint16_t*>(vs.data())[i] = f_to_bf16(vc[i]);
                } else {
                    reinterpret_cast<float*>(ks.data())[i] = kc[i];
                    reinterpret_cast<float*>(vs.data())[i] = vc[i];
                }
            }
    const int32_t n0 = n - 1, zero = 0;
    Tmp dq, dk, dv, dn, dstart, dout, dst;
    OCK(up(dq, qkv.data(), qkv.size() * 4));
    OCK(up(dk, ks.data(), ks.size()));
    OCK(up(dv, vs.data(), vs.size()));
    OCK(up(dn, &n0, 4));
    OCK(up(dstart, &zero, 4));
    OCK(up(dout, nullptr, (size_t)d * 4));
    OCK(up(dst, &zero, 4));
    EngramArgs a{};
    a.qkv = dq.as<float>(); a.k = dk.p; a.v = dv.p; a.n = dn.as<int32_t>(); a.start = dstart.as<int32_t>();
    a.M = 1; a.d = d; a.hs = hs; a.cap = n; a.keep = n; a.bf16 = bf16_store; a.o = dout.as<float>(); a.status = dst.as<uint32_t>();
    if (!launch_engram(0, a, n)) return AVA_ERR_CAPACITY;
    if ((rc = end_())) return rc;
    OCK(cudaMemcpy(out, dout.p, (size_t)d * 4, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

int ava_op_math(int device, int32_t which, const float* x, int64_t n, float* y) {
    if (!x || !y || n <= 0 || which < 0 || which > 2) return AVA_ERR_ARG;
    int rc = begin(device);
    if (rc) return rc;
    Tmp dx, dy;
    OCK(up(dx, x, (size_t)n * 4));
    OCK(up(dy, nullptr, (size_t)n * 4));
    launch_math(0, which, dx.as<float>(), n, dy.as<float>());
    if ((rc = end_())) return rc;
    OCK(cudaMemcpy(y, dy.p, (size_t)n * 4, cudaMemcpyDeviceToHost));
    return AVA_OK;
}

}  // extern "C"
