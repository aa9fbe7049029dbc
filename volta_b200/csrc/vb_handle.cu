// Training handle of libvolta_b200: one device arena, a fixed launch schedule captured as a
// CUDA graph, and the C ABI on top of it.
//
// The step restates volta_train_step of the reference's generated library
// (src/engine/ir/codegen/mlp_train_rust_codegen.rs:699-994) for a GPU:
//   forward   i = 0..n-1   GEMM(act_i, W_i) with bias + activation in the epilogue  (:708-743)
//   loss                    MSE sum and seed gradient                                 (:793-798)
//   backward  i = n-1..0   dW_i = act_i^T.delta_i ; db_i = colsum(delta_i) ;
//                           delta_{i-1} = (delta_i.W_i^T) * f'(.) in the dX epilogue   (:820-934, 958-988)
//   update                  one fused optimizer pass over all parameters              (:958-993)
// All dX GEMMs read W before any update, as in the reference, because the single
// optimizer launch comes last.  Under data parallelism each layer's dW bucket is
// all-reduced on a side stream as soon as it is produced, overlapping the remaining
// backward GEMMs; the optimizer waits for every bucket.
#include <math.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "vb_arena.h"
#include "vb_common.cuh"
#include "vb_checkpoint.h"
#include "vb_dp.h"

using namespace vb;

namespace {

std::mutex g_err_mutex;
std::string g_create_error;
int g_create_status = VB200_OK;

struct KernelRecord {
    std::string name;
    double flops, bytes;
    cudaEvent_t e0, e1;
};

}  // namespace

struct vb200_handle {
    vb200_config cfg;
    int n = 0;  // weight layers
    std::vector<int> L;
    int B = 0;
    long long global_nt = 0;
    int world = 1, rank = 0;
    int status = VB200_OK;
    std::string error;

    ArenaPlan plan;
    char *arena = nullptr;
    int64_t arena_bytes = 0;

    // flat parameter layout (floats): all weights, then all biases, each padded to 64 floats
    std::vector<int64_t> off_w, off_b;
    int64_t n_weights_padded = 0, n_params_padded = 0;
    float *params = nullptr, *grads = nullptr, *s1 = nullptr, *s2 = nullptr;
    float *loss_sum = nullptr;  // lives right behind the gradients so that it joins the bias bucket
    StepScalars *scalars = nullptr;
    unsigned int *status_word = nullptr;
    float *mse_scratch = nullptr, *colsum_scratch = nullptr, *gemm_scratch = nullptr;
    long long gemm_scratch_floats = 0;
    float *xin[2] = {nullptr, nullptr}, *yin[2] = {nullptr, nullptr};
    std::vector<float *> act, pre, delta;  // act[0] unused (slot dependent)

    // optional stages (softmax hidden activation, LayerNorm, dropout, clip); all off in the benchmark configurations
    bool row_opts = false;       // any stage that needs the row kernels
    bool keep_pre = false;       // backward takes the pre-activation from its own buffer
    bool layernorm = false;
    float dropout_p = 0.0f, clip = 0.0f;
    int64_t ln_floats = 0;                   // all gamma/beta blocks, each [gamma(c) | beta(c)] padded to 64 floats
    std::vector<int64_t> off_ln;             // per hidden layer, in floats
    float *ln_params = nullptr, *ln_grads = nullptr, *clip_norm = nullptr;
    std::vector<float *> ln_is;              // per hidden layer [batch]
    std::vector<unsigned char *> mask;       // per hidden layer [batch x c]
    unsigned long long dropout_rng = 12345678ULL;   // mask stream position before the next step (:612, 773)
    unsigned long long draws_per_step = 0;
    std::vector<unsigned long long> draw_off;       // draws of a step that precede this rank's rows of layer k
    cudaEvent_t ev_clip[2] = {nullptr, nullptr};

    // host side
    float *mirror_params = nullptr, *mirror_grads = nullptr;  // pinned
    float *host_loss = nullptr;                               // pinned, one float per slot
    unsigned int *host_status = nullptr;                      // pinned
    // non-finite guard (config check_finite): smallest bad index per region [grads+loss, params, state1, state2]
    bool check_finite = false;
    unsigned long long *first_bad = nullptr, *host_first_bad = nullptr;   // device (arena) / pinned
    unsigned long long wait_ns = 4000000000ull;               // limit of the data-parallel barrier waits
    uint64_t adam_step = 0;
    uint64_t steps_done = 0;
    int last_slot = 0;

    cudaStream_t stream = nullptr, copy_stream = nullptr, comm_stream = nullptr;
    cudaEvent_t ev_copied[2] = {nullptr, nullptr}, ev_slot_free[2] = {nullptr, nullptr};
    cudaEvent_t ev_join = nullptr;
    std::vector<cudaEvent_t> ev_bucket;
    cudaGraphExec_t graph[2] = {nullptr, nullptr};
    // Large HOST inputs: the rows arrive in `in_chunks` copies, and the forward pass (row-independent) runs as one
    // captured graph per chunk as soon as that chunk has landed, followed by the graph of the rest of the step
    static constexpr int kMaxInChunks = 8;
    int in_chunks = 1;
    bool chunked_now = false;     // the step being enqueued takes the chunked path
    bool profiling_next = false;  // the step being enqueued is a profiled one (plain launches, whole forward)
    cudaGraphExec_t graph_fwd[2][kMaxInChunks] = {};
    cudaGraphExec_t graph_rest[2] = {nullptr, nullptr};
    cudaEvent_t ev_chunk[2][kMaxInChunks] = {};
    // inference: pinned staging for host callers and one captured forward graph per row count
    float *infer_in = nullptr, *infer_out = nullptr;
    std::map<long long, cudaGraphExec_t> infer_graphs;
    bool use_graph = true;
    bool fuse_sgd = false;   // plain SGD on one GPU: dW GEMMs update W in their epilogue
    // the whole step as one persistent kernel (batches of at most 64 rows on one GPU; vb_step_small.cu)
    bool small_step = false;
    bool ss_forward = false;   // the same kernel, forward only, serves inference of 9..64 rows
    StepScalars ss_scalars{};  // this step's scalars, handed to the persistent kernel by value
    const float *ss_x = nullptr, *ss_y = nullptr;   // device-resident inputs of this step, used where they lie
    int ss_grid = 0, ss_cluster = 0;
    unsigned int *grid_barrier = nullptr;   // {arrivals, generation, abort} in the arena
    int kernels_per_step = 0;

    DpComm *dp = nullptr;
    // fused data parallelism over peer memory (after volta_b200_dp_attach_peers)
    bool dp_fused = false;
    // exchange by copy (dp_exchange = VB200_DP_PEER_COPY, after attach): one receive slot per rank in the arena
    bool dp_copy = false;
    float *recv = nullptr;
    long long off_recv = 0, recv_slot_floats = 0;
    std::vector<cudaEvent_t> ev_dx;
    PeerTable peers{};
    std::vector<void *> peer_mappings;   // cudaIpcOpenMemHandle results to close
    long long off_params = 0, off_grads = 0, off_s1 = 0, off_s2 = 0, off_flags = 0, off_loss = 0;  // bytes in the arena

    // profiling (plain launches with an event pair per kernel)
    bool profiling = false;
    std::vector<KernelRecord> records;

    // a failure of the handle itself (CUDA, NCCL, a device-side wait): stays in `status`
    int fail(int code, const std::string &msg) {
        status = code;
        error = msg;
        return code;
    }
    // a refused call (bad argument): reported to the caller, the handle stays healthy
    int reject(int code, const std::string &msg) {
        error = msg;
        return code;
    }
};

namespace {

#define VB_CUDA(h, expr)                                                                              \
    do {                                                                                              \
        cudaError_t _e = (expr);                                                                      \
        if (_e != cudaSuccess)                                                                        \
            return (h)->fail(_e == cudaErrorMemoryAllocation ? VB200_ERR_OOM : VB200_ERR_CUDA,        \
                             std::string(#expr) + ": " + cudaGetErrorString(_e));                     \
    } while (0)

int64_t pad64(int64_t v) { return (v + 63) / 64 * 64; }

int pos_fwd(int i) { return i; }
int pos_loss(int n) { return n; }
int pos_bwd(int n, int i) { return n + 1 + (n - 1 - i); }

bool cfg_row_opts(const vb200_config &c) {
    return c.activation == VB200_ACT_SOFTMAX || c.use_layernorm == 1 || c.dropout_p > 0.0f;
}
// Backward needs the pre-activation in a buffer of its own: always for silu/gelu; for relu/leaky
// once LayerNorm or dropout change the stored output, whose sign then no longer tells pre > 0.
// Sigmoid/tanh (and softmax) differentiate through the stored output in the reference (:898-912).
bool cfg_keep_pre(const vb200_config &c) {
    if (act_needs_pre(c.activation)) return true;
    const bool changed = c.use_layernorm == 1 || c.dropout_p > 0.0f;
    return changed && (c.activation == VB200_ACT_RELU || c.activation == VB200_ACT_LEAKY_RELU);
}

// The reference's LCG-Xavier stream (mlp_train_rust_codegen.rs:630-638, 653-658).
void lcg_xavier(float *w, int64_t n, int r, int c, uint64_t *rng) {
    float lim = sqrtf(6.0f / ((float)r + (float)c));
    for (int64_t i = 0; i < n; ++i) {
        *rng = *rng * 6364136223846793005ULL + 1442695040888963407ULL;
        float f = (float)((*rng >> 11) & ((1ULL << 53) - 1)) / (float)(1ULL << 53);
        w[i] = (f * 2.0f - 1.0f) * lim;
    }
}

struct Scope {
    vb200_handle *h;
    bool on;
    // is_kernel = false: a timed wait (for the gradient exchange), not one of this library's launches
    Scope(vb200_handle *h_, const char *name, double flops, double bytes, bool is_kernel = true) : h(h_), on(h_->profiling) {
        if (is_kernel) h->kernels_per_step++;
        if (!on) return;
        KernelRecord r;
        r.name = name;
        r.flops = flops;
        r.bytes = bytes;
        cudaEventCreate(&r.e0);
        cudaEventCreate(&r.e1);
        cudaEventRecord(r.e0, h->stream);
        h->records.push_back(r);
    }
    ~Scope() {
        if (on) cudaEventRecord(h->records.back().e1, h->stream);
    }
};

cudaError_t run_gemm(vb200_handle *h, int layout, const float *A, const float *Bm, long long m, long long n,
                     long long k, const Epilogue &epi) {
    const int path = h->cfg.gemm_path;
    if (layout == GEMM_NN && path == VB200_GEMM_AUTO && gemv_rows_supported(Bm, m, n, k))
        return launch_gemv_rows(A, Bm, m, n, k, epi, h->stream);
    if (path != VB200_GEMM_FFMA && gemm_tc_supported(layout, A, Bm, m, n, k, epi) &&
        (path == VB200_GEMM_TENSOR || path == VB200_GEMM_TENSOR_PAIR || gemm_prefers_tc(m, n, k))) {
        const bool force_pair = path == VB200_GEMM_TENSOR_PAIR;
        // a GEMM that splits K is two launches (the slab reduction follows it): count both
        const int splits = gemm_tc_splits(layout, m, n, k, force_pair);
        if (splits > 1 && h->gemm_scratch_floats >= (long long)splits * m * n) h->kernels_per_step++;
        return launch_gemm_tc(layout, A, Bm, m, n, k, epi, h->status_word, h->stream, h->gemm_scratch,
                              h->gemm_scratch_floats, force_pair);
    }
    if (h->gemm_scratch && ffma_splits(m, n, k) > 1) h->kernels_per_step++;   // likewise on the FFMA path
    return launch_gemm_ffma(layout, A, Bm, m, n, k, epi, h->stream, h->gemm_scratch);
}

int enqueue_small_step(vb200_handle *h, int slot, int rows = 0);

// Forward pass over the first `rows` rows of input slot `slot` (rows <= batch): every layer's GEMM
// with bias and activation fused.  Used by the training step (rows = batch) and by inference.
int enqueue_forward(vb200_handle *h, int slot, long long rows, bool training, const float *in_override = nullptr,
                    float *out_override = nullptr, long long row0 = 0) {
    const int n = h->n, act = h->cfg.activation;
    const long long B = rows;
    const std::vector<int> &L = h->L;
    cudaStream_t s = h->stream;
    // row0 > 0: rows [row0, row0 + rows) of the batch (plain layers only: no row stage keeps per-row state)
    const float *act0 = (in_override ? in_override : h->xin[slot]) + row0 * L[0];
    float *const last_out = (out_override ? out_override : h->act[n]) + row0 * L[n];
    auto A = [&](int i) -> float * { return i == 0 ? const_cast<float *>(act0) : h->act[i] + row0 * L[i]; };
    char nm[64];
    // inference of 9..64 rows: the persistent kernel's forward half, one launch (fewer rows take the
    // cluster kernel below, layer by layer, straight from and to pinned memory)
    if (!training && h->ss_forward && rows > 8 && rows <= 64 && !in_override && !out_override) {
        const int saved = h->kernels_per_step;
        int rc = enqueue_small_step(h, slot, (int)rows);
        h->kernels_per_step = saved;
        return rc;
    }
    for (int i = 0; i < n; ++i) {
        const long long r = L[i], c = L[i + 1];
        Epilogue e{};
        e.act = act;
        e.ld = c;
        e.bias = h->params + h->off_b[i];
        if (i == n - 1) {
            e.mode = EPI_BIAS;
            e.out0 = last_out;
        } else if (act == VB200_ACT_SOFTMAX) {
            e.mode = EPI_BIAS;  // the row kernel below turns the pre-activations into their softmax in place
            e.out0 = h->act[i + 1] + row0 * c;
        } else {
            e.mode = EPI_BIAS_ACT;
            e.out0 = h->act[i + 1] + row0 * c;
            e.out1 = h->keep_pre ? h->pre[i] + row0 * c : nullptr;
        }
        if (i == n - 1 && c == 1) {
            // width-one output layer: a row-dot, bandwidth-bound on act_i
            snprintf(nm, sizeof nm, "fwd%d_rowdot_%lldx%lld", i, B, r);
            Scope sc(h, nm, 2.0 * B * r, 4.0 * (B * r + r + B));
            VB_CUDA(h, launch_rowdot(last_out, A(i), h->params + h->off_w[i], e.bias, B, r, s));
            continue;
        }
        snprintf(nm, sizeof nm, "fwd%d_gemm_nn_%lldx%lldx%lld", i, B, c, r);
        Scope sc(h, nm, 2.0 * B * r * c, 4.0 * (B * r + r * c + B * c * (e.out1 ? 2 : 1)));
        VB_CUDA(h, run_gemm(h, GEMM_NN, A(i), h->params + h->off_w[i], B, c, r, e));
        const bool drop = training && h->dropout_p > 0.0f;
        if (i < n - 1 && (act == VB200_ACT_SOFTMAX || h->layernorm || drop)) {
            RowFwd o{};
            o.softmax = act == VB200_ACT_SOFTMAX;
            if (h->layernorm) {
                o.ln_g = h->ln_params + h->off_ln[i];
                o.ln_b = o.ln_g + c;
                o.ln_is = h->ln_is[i];
            }
            if (drop) {
                o.dropout_p = h->dropout_p;
                o.mask = h->mask[i];
                o.draw_off = h->draw_off[i];
            }
            snprintf(nm, sizeof nm, "fwd%d_rows_%lldx%lld", i, B, c);
            Scope sc(h, nm, 0.0, (8.0 + (drop ? 1.0 : 0.0)) * B * c);
            VB_CUDA(h, launch_row_forward(h->act[i + 1], B, (int)c, o, h->scalars, s));
        }
    }
    return VB200_OK;
}

// Enqueue one whole step on h->stream reading inputs from `slot`.
// Tail of every step: the optional non-finite guard, then loss and status word to pinned memory.
int enqueue_step_tail(vb200_handle *h, int slot) {
    cudaStream_t s = h->stream;
    if (h->check_finite) {
        const int opt = h->cfg.optimizer;
        const bool has1 = opt != VB200_OPT_SGD, has2 = (opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW);
        Scope sc(h, "finite_guard", 0.0, 4.0 * h->n_params_padded * (2 + (has1 ? 1 : 0) + (has2 ? 1 : 0)));
        VB_CUDA(h, cudaMemsetAsync(h->first_bad, 0xFF, 4 * sizeof(unsigned long long), s));
        // the gradient region carries the loss sum right behind it (one more float, or two when the fused
        // data-parallel path keeps the all-rank total beside the local sum)
        VB_CUDA(h, launch_finite_guard(h->params, h->grads, has1 ? h->s1 : nullptr, has2 ? h->s2 : nullptr,
                                       h->n_params_padded, h->n_params_padded + ((h->dp_fused || h->dp_copy) ? 2 : 1), h->first_bad, s));
        VB_CUDA(h, cudaMemcpyAsync(h->host_first_bad, h->first_bad, 4 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s));
    }
    if (h->small_step) return VB200_OK;   // the persistent kernel stores loss and status into pinned memory itself
    VB_CUDA(h, cudaMemcpyAsync(&h->host_loss[slot], (h->dp_fused || h->dp_copy) ? h->loss_sum + 1 : h->loss_sum, sizeof(float),
                               cudaMemcpyDeviceToHost, s));
    VB_CUDA(h, cudaMemcpyAsync(h->host_status, h->status_word, sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
    return VB200_OK;
}

// One launch for the whole step: forward, loss, backward and update inside one persistent kernel
// (rows = batch), or for the forward pass alone (inference of `rows` rows).
int enqueue_small_step(vb200_handle *h, int slot, int rows) {
    const int n = h->n, B = rows > 0 ? rows : h->B;
    const std::vector<int> &L = h->L;
    if (rows == 0) h->kernels_per_step = 0;
    SmallStepArgs a{};
    a.n = n;
    a.B = B;
    a.forward_only = rows > 0 ? 1 : 0;
    a.act = h->cfg.activation;
    a.opt = h->cfg.optimizer;
    a.params = h->params;
    a.grads = h->grads;
    a.s1 = h->s1;
    a.s2 = h->s2;
    a.n_params_padded = h->n_params_padded;
    a.y = h->ss_y ? h->ss_y : h->yin[slot];
    a.loss_sum = h->loss_sum;
    a.loss_partials = h->mse_scratch;
    a.nt_global = (float)h->global_nt;
    a.scalars = h->ss_scalars;
    a.barrier = h->grid_barrier;
    a.status = h->status_word;
    a.host_loss = rows > 0 ? nullptr : &h->host_loss[slot];
    a.host_status = rows > 0 ? nullptr : h->host_status;
    double flops = 0.0;
    for (int i = 0; i < n; ++i) {
        SmallStepLayer &l = a.L[i];
        l.r = L[i];
        l.c = L[i + 1];
        l.off_w = h->off_w[i];
        l.off_b = h->off_b[i];
        l.act_in = i == 0 ? (h->ss_x && rows == 0 ? h->ss_x : h->xin[slot]) : h->act[i];
        l.act_out = h->act[i + 1];
        l.pre_out = (i < n - 1 && h->keep_pre) ? h->pre[i] : nullptr;
        l.delta = h->delta[i];
        l.saved_prev = i == 0 ? nullptr : (h->keep_pre ? h->pre[i - 1] : h->act[i]);
        l.delta_prev = i == 0 ? nullptr : h->delta[i - 1];
        flops += 2.0 * B * L[i] * L[i + 1] * (i == 0 ? 2.0 : 3.0);
    }
    const int opt = h->cfg.optimizer;
    const double bpp = opt == VB200_OPT_SGD ? 16.0 : (opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW) ? 32.0 : 24.0;
    {
        // compulsory traffic: W read forward, then W / state read and W / state / gradient written once
        Scope sc(h, rows > 0 ? "small_forward" : "small_step", flops, bpp * h->n_params_padded);
        VB_CUDA(h, launch_small_step(a, h->ss_grid, h->ss_cluster, h->stream));
    }
    return rows > 0 ? VB200_OK : enqueue_step_tail(h, slot);
}

// skip_forward: the forward pass has been enqueued already (in row chunks, see in_chunks).
int enqueue_step(vb200_handle *h, int slot, bool skip_forward = false) {
    if (h->small_step) return enqueue_small_step(h, slot);
    const int n = h->n, B = h->B, act = h->cfg.activation;
    const std::vector<int> &L = h->L;
    cudaStream_t s = h->stream;
    h->kernels_per_step = 0;
    const float *act0 = h->xin[slot];
    auto A = [&](int i) -> float * { return i == 0 ? const_cast<float *>(act0) : h->act[i]; };
    char nm[64];

    if (!skip_forward) {
        int rc = enqueue_forward(h, slot, B, true);
        if (rc) return rc;
    }
    // loss + seed gradient
    {
        long long nt = (long long)B * L[n];
        Scope sc(h, "mse_seed", 3.0 * nt, 12.0 * nt);
        h->kernels_per_step++;  // two launches
        VB_CUDA(h, launch_mse_seed(h->delta[n - 1], h->loss_sum, h->act[n], h->yin[slot], nt, (float)h->global_nt,
                                   h->mse_scratch, s));
    }
    // backward.  Per layer: dW_i, db_i, then dX_i -> delta_{i-1}.  With the SGD update folded into
    // the dW epilogue, dX_i (which must read the pre-update W_i) goes first.  With the clip every
    // delta must exist before any dW is taken (:936-955), so the dW GEMMs form a second sweep.
    const bool two_sweeps = h->clip > 0.0f;
    const bool nccl_bucket_update = h->dp && !h->dp_fused && !h->dp_copy && !two_sweeps && !h->layernorm;
    // LayerNorm backward -> dropout mask -> activation backward on the raw delta of hidden layer i
    auto do_rows = [&](int i) -> int {
        if (!h->row_opts || i == n - 1) return VB200_OK;
        const long long c = L[i + 1];
        RowBwd o{};
        o.act = act;
        o.a1 = h->act[i + 1];
        o.saved = h->keep_pre ? h->pre[i] : h->act[i + 1];
        if (h->layernorm) {
            o.ln_g = h->ln_params + h->off_ln[i];
            o.ln_b = o.ln_g + c;
            o.ln_is = h->ln_is[i];
            snprintf(nm, sizeof nm, "ln%d_param_grads_%lldx%lld", i, (long long)B, c);
            Scope sc(h, nm, 3.0 * B * c, 8.0 * B * c);
            h->kernels_per_step++;
            VB_CUDA(h, launch_ln_param_grads(h->ln_grads + h->off_ln[i], h->delta[i], h->act[i + 1], o.ln_g, o.ln_b, B,
                                             (int)c, h->colsum_scratch, s));
        }
        if (h->dropout_p > 0.0f) {
            o.dropout_p = h->dropout_p;
            o.mask = h->mask[i];
        }
        snprintf(nm, sizeof nm, "bwd%d_rows_%lldx%lld", i, (long long)B, c);
        Scope sc(h, nm, 0.0, 16.0 * B * c);
        VB_CUDA(h, launch_row_backward(h->delta[i], B, (int)c, o, s));
        return VB200_OK;
    };
    auto do_dx = [&](int i) -> int {
        if (i == 0) return VB200_OK;
        const long long r = L[i], c = L[i + 1];
        Epilogue e{};
        e.act = act;
        e.out0 = h->delta[i - 1];
        e.ld = r;
        if (h->row_opts) {
            e.mode = EPI_STORE;  // do_rows(i - 1) finishes this delta
        } else {
            e.mode = EPI_DACT;
            e.saved = h->keep_pre ? h->pre[i - 1] : h->act[i];
        }
        if (c == 1 && h->cfg.gemm_path == VB200_GEMM_AUTO) {
            // width-one layer: the product is an outer product, one streaming pass
            snprintf(nm, sizeof nm, "dX%d_rank1_%lldx%lld", i, (long long)B, r);
            Scope sc(h, nm, 2.0 * B * r, 4.0 * (B + r + 2.0 * B * r));
            VB_CUDA(h, launch_rank1_dx(e.out0, h->delta[i], h->params + h->off_w[i], e.mode == EPI_DACT ? e.saved : nullptr, act,
                                       B, r, s));
            return VB200_OK;
        }
        snprintf(nm, sizeof nm, "dX%d_gemm_nt_%lldx%lldx%lld", i, (long long)B, r, c);
        Scope sc(h, nm, 2.0 * B * r * c, 4.0 * (B * c + r * c + 2.0 * B * r));
        VB_CUDA(h, run_gemm(h, GEMM_NT, h->delta[i], h->params + h->off_w[i], B, r, c, e));
        return VB200_OK;
    };
#define VB_TRY(call)          \
    do {                      \
        int _rc = (call);     \
        if (_rc) return _rc;  \
    } while (0)
    // exchange by copy: floats [begin, begin + count) of this rank's gradient region go into slot `rank` of every
    // other rank's arena, nearest higher rank first, so that at any moment the ranks write to different peers
    auto push_to_peers = [&](long long begin, long long count) -> int {
        for (int d = 1; d < h->world; ++d) {
            const int p = (h->rank + d) % h->world;
            char *dst = h->peers.base[p] + h->off_recv + ((long long)h->rank * h->recv_slot_floats + begin) * 4;
            VB_CUDA(h, cudaMemcpyAsync(dst, h->grads + begin, (size_t)count * 4, cudaMemcpyDeviceToDevice, h->comm_stream));
        }
        return VB200_OK;
    };
    auto do_dw = [&](int i) -> int {
        const long long r = L[i], c = L[i + 1];
        const bool fused = h->fuse_sgd && c != 1;
        if (c == 1) {
            // dW of a width-one layer: column sums of act_i weighted by delta_i[row]
            snprintf(nm, sizeof nm, "dW%d_wcolsum_%lldx%lld", i, (long long)B, r);
            Scope sc(h, nm, 2.0 * B * r, 4.0 * (B * r + B + r));
            h->kernels_per_step++;
            VB_CUDA(h, launch_colsum(h->grads + h->off_w[i], A(i), B, r, h->colsum_scratch, s, h->delta[i]));
        } else {
            Epilogue e{};
            e.mode = fused ? EPI_SGD : EPI_STORE;
            e.out0 = fused ? h->params + h->off_w[i] : h->grads + h->off_w[i];
            e.lr = &h->scalars->lr;
            e.ld = c;
            snprintf(nm, sizeof nm, fused ? "dW%d_sgd_gemm_tn_%lldx%lldx%lld" : "dW%d_gemm_tn_%lldx%lldx%lld", i, r, c, (long long)B);
            Scope sc(h, nm, 2.0 * B * r * c, 4.0 * (B * r + B * c + (fused ? 2.0 : 1.0) * r * c));
            VB_CUDA(h, run_gemm(h, GEMM_TN, A(i), h->delta[i], r, c, B, e));
        }
        if (h->dp_copy) {
            // bucket i = dW_i: the copy engines push it into this rank's slot of every peer while the main stream goes on
            VB_CUDA(h, cudaEventRecord(h->ev_bucket[i], s));
            VB_CUDA(h, cudaStreamWaitEvent(h->comm_stream, h->ev_bucket[i], 0));
            VB_TRY(push_to_peers(h->off_w[i], pad64(r * c)));
        } else if (h->dp && !h->dp_fused) {
            // bucket i = dW_i: reduce on the side stream while the main stream goes on
            VB_CUDA(h, cudaEventRecord(h->ev_bucket[i], s));
            VB_CUDA(h, cudaStreamWaitEvent(h->comm_stream, h->ev_bucket[i], 0));
            int rc = h->dp->all_reduce_sum(h->grads + h->off_w[i], pad64(r * c), h->comm_stream);
            if (rc) return h->fail(VB200_ERR_NCCL, h->dp->error());
        }
        return VB200_OK;
    };
    auto do_db = [&](int i) -> int {
        const long long c = L[i + 1];
        snprintf(nm, sizeof nm, "db%d_colsum_%lldx%lld", i, (long long)B, c);
        Scope sc(h, nm, (double)B * c, 4.0 * (B * c + c));
        h->kernels_per_step++;
        VB_CUDA(h, launch_colsum(h->grads + h->off_b[i], h->delta[i], B, c, h->colsum_scratch, s));
        return VB200_OK;
    };
    for (int i = n - 1; i >= 0; --i) {
        const long long r = L[i], c = L[i + 1];
        VB_TRY(do_rows(i));
        if (two_sweeps) {
            VB_TRY(do_db(i));
            VB_TRY(do_dx(i));
            continue;
        }
        const bool fused = h->fuse_sgd && c != 1;
        if (fused) VB_TRY(do_dx(i));
        // the first layer's bias gradient goes ahead of its dW, so that behind the step's last GEMM only that
        // GEMM's own bucket is left to exchange
        if (i == 0 && h->dp) VB_TRY(do_db(i));
        VB_TRY(do_dw(i));
        if (!(i == 0 && h->dp)) VB_TRY(do_db(i));
        if (!fused) VB_TRY(do_dx(i));
        if (nccl_bucket_update) {
            // NCCL buckets: once this rank is past dX_i (nothing reads W_i any more) the bucket's optimizer pass
            // follows its all-reduce on the side stream, underneath the remaining backward GEMMs
            const int opt = h->cfg.optimizer;
            const bool has1 = opt != VB200_OPT_SGD, has2 = opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW;
            VB_CUDA(h, cudaEventRecord(h->ev_dx[i], s));
            VB_CUDA(h, cudaStreamWaitEvent(h->comm_stream, h->ev_dx[i], 0));
            h->kernels_per_step++;
            VB_CUDA(h, launch_optimizer(opt, h->params + h->off_w[i], has1 ? h->s1 + h->off_w[i] : h->s1,
                                        has2 ? h->s2 + h->off_w[i] : h->s2, h->grads + h->off_w[i], pad64(r * c), pad64(r * c),
                                        h->scalars, h->comm_stream));
        }
        if (h->dp_copy) {
            // bucket i, on the side stream: once this rank is past dX_i (nothing reads W_i any more) and a barrier
            // shows that every rank's push of the bucket has landed, add the copies and update W_i
            VB_CUDA(h, cudaEventRecord(h->ev_dx[i], s));
            VB_CUDA(h, cudaStreamWaitEvent(h->comm_stream, h->ev_dx[i], 0));
            h->kernels_per_step += 2;
            VB_CUDA(h, launch_dp_barrier(h->peers, h->off_flags, h->world, h->rank, h->scalars, (unsigned)(n + 2),
                                         (unsigned)(n - i), h->status_word, h->wait_ns, h->comm_stream));
            VB_CUDA(h, launch_dp_gather_update(h->cfg.optimizer, h->params, h->s1, h->s2, h->grads, h->recv, h->recv_slot_floats,
                                               h->off_w[i], pad64(r * c), h->n_weights_padded, h->world, h->rank, h->scalars,
                                               -1, h->status_word, h->comm_stream));
        }
        if (h->dp_fused) {
            // bucket i over peer memory, on the side stream: once EVERY rank is past dX_i (nobody reads
            // W_i any more, every dW_i is final) reduce + update + redistribute W_i in one kernel
            VB_CUDA(h, cudaEventRecord(h->ev_bucket[i], s));
            VB_CUDA(h, cudaStreamWaitEvent(h->comm_stream, h->ev_bucket[i], 0));
            h->kernels_per_step += 2;
            VB_CUDA(h, launch_dp_barrier(h->peers, h->off_flags, h->world, h->rank, h->scalars, (unsigned)(n + 2),
                                         (unsigned)(n - i), h->status_word, h->wait_ns, h->comm_stream));
            VB_CUDA(h, launch_dp_reduce_update(h->cfg.optimizer, h->peers, h->off_params, h->off_grads, h->off_s1, h->off_s2,
                                               h->off_w[i], pad64(r * c), h->n_weights_padded, h->world, h->rank,
                                               h->scalars, -1, h->status_word, h->comm_stream));
        }
    }
    if (two_sweeps) {
        // norm over every delta (all ranks' rows under data parallelism), then scale, then the dW sweep
        long long nb = 0;
        {
            Scope sc(h, "clip_norm", 0.0, 0.0);
            for (int i = 0; i < n; ++i) {
                const long long cnt = (long long)B * L[i + 1];
                h->kernels_per_step++;
                VB_CUDA(h, launch_sumsq_partials(h->mse_scratch + nb, h->delta[i], cnt, s));
                nb += loss_blocks(cnt);
            }
            VB_CUDA(h, launch_sum_partials(h->clip_norm, h->mse_scratch, nb, s));
        }
        if (h->dp) {
            VB_CUDA(h, cudaEventRecord(h->ev_clip[0], s));
            VB_CUDA(h, cudaStreamWaitEvent(h->comm_stream, h->ev_clip[0], 0));
            int rc = h->dp->all_reduce_sum(h->clip_norm, 64, h->comm_stream);
            if (rc) return h->fail(VB200_ERR_NCCL, h->dp->error());
            VB_CUDA(h, cudaEventRecord(h->ev_clip[1], h->comm_stream));
            VB_CUDA(h, cudaStreamWaitEvent(s, h->ev_clip[1], 0));
        }
        {
            Scope sc(h, "clip_scale", 0.0, 0.0);
            h->kernels_per_step += n - 1;
            for (int i = 0; i < n; ++i)
                VB_CUDA(h, launch_clip_scale(h->delta[i], (long long)B * L[i + 1], h->clip_norm, h->clip, s));
        }
        for (int i = n - 1; i >= 0; --i) VB_TRY(do_dw(i));
    }
#undef VB_TRY
    if (h->dp_fused) {
        // last bucket: all biases, and the loss; then one barrier so that every update has landed
        // everywhere before the step ends
        VB_CUDA(h, cudaEventRecord(h->ev_bucket[n], s));
        VB_CUDA(h, cudaStreamWaitEvent(h->comm_stream, h->ev_bucket[n], 0));
        h->kernels_per_step += 3;
        VB_CUDA(h, launch_dp_barrier(h->peers, h->off_flags, h->world, h->rank, h->scalars, (unsigned)(n + 2),
                                     (unsigned)(n + 1), h->status_word, h->wait_ns, h->comm_stream));
        VB_CUDA(h, launch_dp_reduce_update(h->cfg.optimizer, h->peers, h->off_params, h->off_grads, h->off_s1, h->off_s2,
                                           h->n_weights_padded, h->n_params_padded - h->n_weights_padded,
                                           h->n_weights_padded, h->world, h->rank, h->scalars, h->off_loss, h->status_word,
                                           h->comm_stream));
        VB_CUDA(h, launch_dp_barrier(h->peers, h->off_flags, h->world, h->rank, h->scalars, (unsigned)(n + 2),
                                     (unsigned)(n + 2), h->status_word, h->wait_ns, h->comm_stream));
        VB_CUDA(h, cudaEventRecord(h->ev_join, h->comm_stream));
        VB_CUDA(h, cudaStreamWaitEvent(s, h->ev_join, 0));
    }
    if (h->dp_copy) {
        // last bucket: every bias gradient and the loss sum; then one barrier so that no rank starts the next
        // step's pushes while another still reads its receive slots
        VB_CUDA(h, cudaEventRecord(h->ev_bucket[n], s));
        VB_CUDA(h, cudaStreamWaitEvent(h->comm_stream, h->ev_bucket[n], 0));
        const long long nb = h->n_params_padded - h->n_weights_padded;
        {
            int rc = push_to_peers(h->n_weights_padded, nb + 64);
            if (rc) return rc;
        }
        h->kernels_per_step += 3;
        VB_CUDA(h, launch_dp_barrier(h->peers, h->off_flags, h->world, h->rank, h->scalars, (unsigned)(n + 2),
                                     (unsigned)(n + 1), h->status_word, h->wait_ns, h->comm_stream));
        VB_CUDA(h, launch_dp_gather_update(h->cfg.optimizer, h->params, h->s1, h->s2, h->grads, h->recv, h->recv_slot_floats,
                                           h->n_weights_padded, nb, h->n_weights_padded, h->world, h->rank, h->scalars,
                                           h->n_params_padded, h->status_word, h->comm_stream));
        VB_CUDA(h, launch_dp_barrier(h->peers, h->off_flags, h->world, h->rank, h->scalars, (unsigned)(n + 2),
                                     (unsigned)(n + 2), h->status_word, h->wait_ns, h->comm_stream));
        VB_CUDA(h, cudaEventRecord(h->ev_join, h->comm_stream));
        Scope sc(h, "wait_for_gradient_exchange", 0.0, 0.0, false);
        VB_CUDA(h, cudaStreamWaitEvent(s, h->ev_join, 0));
    }
    if (h->dp && !h->dp_fused && !h->dp_copy) {
        // last bucket: every bias gradient plus the loss sum, contiguous behind the weights
        VB_CUDA(h, cudaEventRecord(h->ev_bucket[n], s));
        VB_CUDA(h, cudaStreamWaitEvent(h->comm_stream, h->ev_bucket[n], 0));
        // (and the LayerNorm gradients, which follow the loss slot)
        int64_t cnt = h->n_params_padded - h->n_weights_padded + 64 + h->ln_floats;
        int rc = h->dp->all_reduce_sum(h->grads + h->n_weights_padded, cnt, h->comm_stream);
        if (rc) return h->fail(VB200_ERR_NCCL, h->dp->error());
        VB_CUDA(h, cudaEventRecord(h->ev_join, h->comm_stream));
        // what of the exchange is NOT hidden under the backward GEMMs shows up as this wait
        Scope sc(h, "wait_for_gradient_exchange", 0.0, 0.0, false);
        VB_CUDA(h, cudaStreamWaitEvent(s, h->ev_join, 0));
    }
    // update
    {
        const int opt = h->cfg.optimizer;
        double bpp = opt == VB200_OPT_SGD ? 12.0 : (opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW) ? 28.0 : 20.0;
        if (h->dp_fused || h->dp_copy) {
            // every parameter was updated inside the bucket kernels
        } else if (h->fuse_sgd) {
            // weights of every layer wider than one were updated by their dW GEMM; the rest follows here
            for (int i = 0; i < n; ++i)
                if (L[i + 1] == 1) {
                    Scope sc(h, "optimizer_w1", 0.0, bpp * L[i]);
                    VB_CUDA(h, launch_optimizer(opt, h->params + h->off_w[i], h->s1, h->s2, h->grads + h->off_w[i],
                                                pad64(L[i]), 0, h->scalars, s));
                }
            const int64_t nb = h->n_params_padded - h->n_weights_padded;
            Scope sc(h, "optimizer_bias", 0.0, bpp * nb);
            VB_CUDA(h, launch_optimizer(opt, h->params + h->n_weights_padded, h->s1, h->s2, h->grads + h->n_weights_padded,
                                        nb, 0, h->scalars, s));
        } else if (nccl_bucket_update) {
            // the weights were updated bucket by bucket on the side stream; the biases follow here
            const bool has1 = opt != VB200_OPT_SGD, has2 = opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW;
            const int64_t w = h->n_weights_padded, nb = h->n_params_padded - w;
            Scope sc(h, "optimizer_bias", 0.0, bpp * nb);
            VB_CUDA(h, launch_optimizer(opt, h->params + w, has1 ? h->s1 + w : h->s1, has2 ? h->s2 + w : h->s2, h->grads + w, nb, 0,
                                        h->scalars, s));
        } else {
            Scope sc(h, "optimizer", 0.0, bpp * h->n_params_padded);
            VB_CUDA(h, launch_optimizer(opt, h->params, h->s1, h->s2, h->grads, h->n_params_padded, h->n_weights_padded,
                                        h->scalars, s));
        }
        if (h->layernorm) {
            // gamma/beta always take a plain SGD step with this step's lr (:876-887).  The reference does it
            // inside the backward sweep; nothing reads them again before the next forward, so it can wait
            // for the (possibly all-reduced) gradients here.
            Scope sc(h, "layernorm_sgd", 0.0, 12.0 * h->ln_floats);
            VB_CUDA(h, launch_optimizer(VB200_OPT_SGD, h->ln_params, nullptr, nullptr, h->ln_grads, h->ln_floats, 0,
                                        h->scalars, s));
        }
    }
    return enqueue_step_tail(h, slot);
}

void destroy_step_graphs(vb200_handle *h) {
    for (int s = 0; s < 2; ++s) {
        if (h->graph[s]) cudaGraphExecDestroy(h->graph[s]);
        if (h->graph_rest[s]) cudaGraphExecDestroy(h->graph_rest[s]);
        h->graph[s] = h->graph_rest[s] = nullptr;
        for (int c = 0; c < vb200_handle::kMaxInChunks; ++c) {
            if (h->graph_fwd[s][c]) cudaGraphExecDestroy(h->graph_fwd[s][c]);
            h->graph_fwd[s][c] = nullptr;
        }
    }
}

// Captures what `body` enqueues on the handle's stream into an executable graph.
template <class Body>
int capture_one(vb200_handle *h, cudaGraphExec_t *out, Body body) {
    cudaGraph_t g = nullptr;
    VB_CUDA(h, cudaStreamBeginCapture(h->stream, cudaStreamCaptureModeThreadLocal));
    int rc = body();
    cudaError_t e = cudaStreamEndCapture(h->stream, &g);
    if (rc) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (e != cudaSuccess) return h->fail(VB200_ERR_CUDA, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(e));
    e = cudaGraphInstantiate(out, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return h->fail(VB200_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
    return VB200_OK;
}

int capture_graphs(vb200_handle *h) {
    for (int slot = 0; slot < 2; ++slot) {
        if (h->in_chunks > 1) {
            // host inputs: one graph per row chunk of the forward pass, one for the rest of the step
            const long long rows = h->B / h->in_chunks;
            for (int c = 0; c < h->in_chunks; ++c) {
                int rc = capture_one(h, &h->graph_fwd[slot][c], [&] { return enqueue_forward(h, slot, rows, true, nullptr, nullptr, c * rows); });
                if (rc) return rc;
            }
            int rc = capture_one(h, &h->graph_rest[slot], [&] { return enqueue_step(h, slot, true); });
            if (rc) return rc;
        }
        int rc = capture_one(h, &h->graph[slot], [&] { return enqueue_step(h, slot); });
        if (rc) return rc;
    }
    return VB200_OK;
}

StepScalars make_scalars(vb200_handle *h, float lr) {
    StepScalars sc{};
    sc.lr = lr;
    sc.beta1 = 0.9f;
    sc.beta2 = 0.999f;
    sc.eps = 1e-8f;
    sc.weight_decay = h->cfg.weight_decay != 0.0f ? h->cfg.weight_decay : 0.01f;
    sc.momentum = h->cfg.momentum != 0.0f ? h->cfg.momentum : 0.9f;
    // mlp_train_rust_codegen.rs:805-811: the counter is bumped before the update and the
    // corrections use f32 powf
    float t = (float)h->adam_step;
    sc.bc1 = 1.0f - powf(sc.beta1, t);
    sc.bc2 = 1.0f - powf(sc.beta2, t);
    sc.epoch = (unsigned int)(h->steps_done + 1);
    sc.rng_base = h->dropout_rng;
    return sc;
}

int copy_inputs(vb200_handle *h, int slot, const float *X, const float *Y, bool *host_wait) {
    const size_t xb = (size_t)h->B * h->L[0] * sizeof(float), yb = (size_t)h->B * h->L[h->n] * sizeof(float);
    cudaPointerAttributes ax{}, ay{};
    cudaError_t ex = cudaPointerGetAttributes(&ax, X), ey = cudaPointerGetAttributes(&ay, Y);
    if (ex != cudaSuccess || ey != cudaSuccess) {
        cudaGetLastError();
        ax.type = cudaMemoryTypeUnregistered;
        ay.type = cudaMemoryTypeUnregistered;
    }
    const bool xdev = ax.type == cudaMemoryTypeDevice || ax.type == cudaMemoryTypeManaged;
    const bool ydev = ay.type == cudaMemoryTypeDevice || ay.type == cudaMemoryTypeManaged;
    // The persistent step kernel takes its input pointers as arguments of each launch: inputs that already
    // live on the device are read where they lie (they must stay unchanged until the step has run), only
    // host inputs go through the slot.
    h->ss_x = (h->small_step && xdev) ? X : nullptr;
    h->ss_y = (h->small_step && ydev) ? Y : nullptr;
    *host_wait = !(xdev && ydev);
    h->chunked_now = h->in_chunks > 1 && !xdev && h->graph_rest[slot] != nullptr && !h->profiling_next;
    if (h->ss_x && h->ss_y) return VB200_OK;
    // the slot is free once the step that last read it has finished
    VB_CUDA(h, cudaStreamWaitEvent(h->copy_stream, h->ev_slot_free[slot], 0));
    if (h->chunked_now) {
        // Y first (small), then X in row chunks with an event behind each: the forward graph of a chunk starts
        // as soon as its rows have landed, while the later chunks are still on their way
        VB_CUDA(h, cudaMemcpyAsync(h->yin[slot], Y, yb, ydev ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice,
                                   h->copy_stream));
        const size_t cb = xb / (size_t)h->in_chunks;
        for (int c = 0; c < h->in_chunks; ++c) {
            VB_CUDA(h, cudaMemcpyAsync(reinterpret_cast<char *>(h->xin[slot]) + c * cb, reinterpret_cast<const char *>(X) + c * cb,
                                       cb, cudaMemcpyHostToDevice, h->copy_stream));
            VB_CUDA(h, cudaEventRecord(h->ev_chunk[slot][c], h->copy_stream));
        }
        VB_CUDA(h, cudaEventRecord(h->ev_copied[slot], h->copy_stream));
        return VB200_OK;
    }
    if (!h->ss_x)
        VB_CUDA(h, cudaMemcpyAsync(h->xin[slot], X, xb, xdev ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice,
                                   h->copy_stream));
    if (!h->ss_y)
        VB_CUDA(h, cudaMemcpyAsync(h->yin[slot], Y, yb, ydev ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice,
                                   h->copy_stream));
    VB_CUDA(h, cudaEventRecord(h->ev_copied[slot], h->copy_stream));
    VB_CUDA(h, cudaStreamWaitEvent(h->stream, h->ev_copied[slot], 0));
    return VB200_OK;
}

// Name of the tensor that holds flat index `idx` of the parameter layout, and the index inside it.
std::string flat_name(const vb200_handle *h, unsigned long long idx, unsigned long long *local) {
    for (int i = 0; i < h->n; ++i) {
        const unsigned long long w0 = (unsigned long long)h->off_w[i], wn = (unsigned long long)h->L[i] * h->L[i + 1];
        if (idx >= w0 && idx < w0 + wn) { *local = idx - w0; return "'layer" + std::to_string(i) + ".weight'"; }
        const unsigned long long b0 = (unsigned long long)h->off_b[i], bn = (unsigned long long)h->L[i + 1];
        if (idx >= b0 && idx < b0 + bn) { *local = idx - b0; return "'layer" + std::to_string(i) + ".bias'"; }
    }
    *local = idx;
    return "(padding)";
}

// What the last finished step left in pinned memory: the status word of the device-side waits and,
// under check_finite, the first non-finite element per region (message as the reference's
// ensure_finite_tensor, src/engine/ir/train.rs:681-701).
int check_device_status(vb200_handle *h) {
    if (h->host_status && *h->host_status != 0) {
        char buf[160];
        snprintf(buf, sizeof buf, "a device-side wait gave up (status word 0x%08x%s)", *h->host_status,
                 (*h->host_status & kStatusDpBarrier) ? ": a data-parallel rank did not reach a barrier in time; no update was applied" : "");
        return h->fail(VB200_ERR_DEVICE_WAIT, buf);
    }
    if (h->check_finite && h->host_first_bad) {
        static const char *kind[4] = {"gradient", "parameter", "optimizer_state.1", "optimizer_state.2"};
        for (int r = 0; r < 4; ++r) {
            const unsigned long long idx = h->host_first_bad[r];
            if (idx == ~0ULL) continue;
            std::string msg;
            if (r == 0 && idx >= (unsigned long long)h->n_params_padded) {
                msg = "Non-finite train loss";
            } else {
                unsigned long long local = 0;
                const std::string name = flat_name(h, idx, &local);
                msg = std::string("Non-finite train ") + kind[r] + " " + name + " at element " + std::to_string(local);
            }
            return h->fail(VB200_ERR_NONFINITE, msg + " (step " + std::to_string((unsigned long long)h->steps_done) + ")");
        }
    }
    return VB200_OK;
}

int do_step(vb200_handle *h, const float *X, const float *Y, float lr, bool profile) {
    if (!X || !Y) return h->reject(VB200_ERR_INVALID, "volta_b200_step: null input pointer");
    // A handle that failed (a device-side wait that ran out, a CUDA or NCCL error, a non-finite value
    // under check_finite) takes no further steps: its state is no longer one the reference could reach,
    // and after a data-parallel wait gave up a peer may be gone.  The status word of the last finished
    // step sits in pinned memory, so looking costs nothing.
    if (h->status != VB200_OK) return h->status;
    {
        int rc0 = check_device_status(h);
        if (rc0) return rc0;
    }
    const int slot = profile ? 0 : (int)(h->steps_done & 1);
    bool host_wait = false;
    h->profiling_next = profile;
    int rc = copy_inputs(h, slot, X, Y, &host_wait);
    h->profiling_next = false;
    if (rc) return rc;
    const int opt = h->cfg.optimizer;
    if (opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW) h->adam_step += 1;
    if (h->small_step) {
        h->ss_scalars = make_scalars(h, lr);   // a kernel argument: no helper launch, no graph
    } else {
        VB_CUDA(h, launch_set_scalars(h->scalars, make_scalars(h, lr), h->stream));
    }
    if (profile || !h->use_graph || h->small_step) {
        h->profiling = profile;
        rc = enqueue_step(h, slot);
        h->profiling = false;
        if (rc) return rc;
    } else if (h->chunked_now) {
        for (int c = 0; c < h->in_chunks; ++c) {
            VB_CUDA(h, cudaStreamWaitEvent(h->stream, h->ev_chunk[slot][c], 0));
            VB_CUDA(h, cudaGraphLaunch(h->graph_fwd[slot][c], h->stream));
        }
        VB_CUDA(h, cudaStreamWaitEvent(h->stream, h->ev_copied[slot], 0));
        VB_CUDA(h, cudaGraphLaunch(h->graph_rest[slot], h->stream));
    } else {
        VB_CUDA(h, cudaGraphLaunch(h->graph[slot], h->stream));
    }
    if (!(h->ss_x && h->ss_y)) VB_CUDA(h, cudaEventRecord(h->ev_slot_free[slot], h->stream));
    h->last_slot = slot;
    h->steps_done += 1;
    if (h->draws_per_step) h->dropout_rng = lcg_jump(h->dropout_rng, h->draws_per_step);
    // X and Y are borrowed for the call only (mlp_train_rust_codegen.rs:704-707 copies X
    // before returning): wait until the device has taken them out of host memory.
    if (host_wait) VB_CUDA(h, cudaEventSynchronize(h->ev_copied[slot]));
    return VB200_OK;
}


void destroy(vb200_handle *h) {
    if (!h) return;
    if (h->stream) cudaStreamSynchronize(h->stream);
    if (h->copy_stream) cudaStreamSynchronize(h->copy_stream);
    if (h->comm_stream) cudaStreamSynchronize(h->comm_stream);
    // The captured graphs hold references on the communicator (NCCL waits for them in its
    // destroy call), so they must go first.
    destroy_step_graphs(h);
    for (auto &kv : h->infer_graphs) cudaGraphExecDestroy(kv.second);
    h->infer_graphs.clear();
    if (h->infer_in) cudaFreeHost(h->infer_in);
    if (h->infer_out) cudaFreeHost(h->infer_out);
    if (h->dp) {
        delete h->dp;
        h->dp = nullptr;
    }
    for (int s = 0; s < 2; ++s) {
        if (h->ev_copied[s]) cudaEventDestroy(h->ev_copied[s]);
        if (h->ev_slot_free[s]) cudaEventDestroy(h->ev_slot_free[s]);
    }
    if (h->ev_join) cudaEventDestroy(h->ev_join);
    for (int q = 0; q < 2; ++q)
        if (h->ev_clip[q]) cudaEventDestroy(h->ev_clip[q]);
    for (auto e : h->ev_bucket) cudaEventDestroy(e);
    for (auto e : h->ev_dx) cudaEventDestroy(e);
    for (int s = 0; s < 2; ++s)
        for (int c = 0; c < vb200_handle::kMaxInChunks; ++c)
            if (h->ev_chunk[s][c]) cudaEventDestroy(h->ev_chunk[s][c]);
    for (void *m : h->peer_mappings) cudaIpcCloseMemHandle(m);
    if (h->arena) cudaFree(h->arena);
    if (h->mirror_params) cudaFreeHost(h->mirror_params);
    if (h->mirror_grads) cudaFreeHost(h->mirror_grads);
    if (h->host_loss) cudaFreeHost(h->host_loss);
    if (h->host_status) cudaFreeHost(h->host_status);
    if (h->host_first_bad) cudaFreeHost(h->host_first_bad);
    if (h->stream) cudaStreamDestroy(h->stream);
    if (h->copy_stream) cudaStreamDestroy(h->copy_stream);
    if (h->comm_stream) cudaStreamDestroy(h->comm_stream);
    delete h;
}

int validate(const vb200_config *c, std::string *why) {
    if (!c) { *why = "null config"; return VB200_ERR_INVALID; }
    if (c->n_sizes < 2 || c->n_sizes > VB200_MAX_LAYERS) { *why = "need between 2 and 32 layer sizes"; return VB200_ERR_INVALID; }
    for (int i = 0; i < c->n_sizes; ++i)
        if (c->layers[i] <= 0) { *why = "layer widths must be positive"; return VB200_ERR_INVALID; }
    if (c->batch <= 0) { *why = "batch must be positive"; return VB200_ERR_INVALID; }
    if (c->activation < VB200_ACT_RELU || c->activation > VB200_ACT_SOFTMAX) { *why = "unknown activation"; return VB200_ERR_UNSUPPORTED; }
    if (!(c->dropout_p >= 0.0f && c->dropout_p < 1.0f)) { *why = "dropout_p must lie in [0, 1)"; return VB200_ERR_INVALID; }
    if (!(c->clip_grad >= 0.0f)) { *why = "clip_grad must not be negative"; return VB200_ERR_INVALID; }
    if (c->use_layernorm != 0 && c->use_layernorm != 1) { *why = "use_layernorm must be 0 or 1"; return VB200_ERR_INVALID; }
    if (cfg_row_opts(*c))
        for (int i = 1; i < c->n_sizes - 1; ++i)
            if (c->layers[i] > kRowMaxCols) { *why = "softmax, LayerNorm and dropout take hidden widths up to 51200"; return VB200_ERR_UNSUPPORTED; }
    if (c->optimizer < VB200_OPT_SGD || c->optimizer > VB200_OPT_SGD_MOMENTUM) { *why = "unknown optimizer"; return VB200_ERR_UNSUPPORTED; }
    int world = c->world_size > 1 ? c->world_size : 1;
    if (c->rank < 0 || c->rank >= world) { *why = "rank out of range"; return VB200_ERR_INVALID; }
    if (c->global_batch != 0 && c->global_batch < c->batch) { *why = "global_batch smaller than batch"; return VB200_ERR_INVALID; }
    if (c->gemm_path < VB200_GEMM_AUTO || c->gemm_path > VB200_GEMM_TENSOR_PAIR) { *why = "unknown gemm_path"; return VB200_ERR_INVALID; }
    if (c->device_wait_ms < 0) { *why = "device_wait_ms must not be negative"; return VB200_ERR_INVALID; }
    if (c->check_finite != 0 && c->check_finite != 1) { *why = "check_finite must be 0 or 1"; return VB200_ERR_INVALID; }
    if (c->step_kernel < 0 || c->step_kernel > 2) { *why = "step_kernel must be 0, 1 or 2"; return VB200_ERR_INVALID; }
    if (c->dp_exchange < VB200_DP_NCCL || c->dp_exchange > VB200_DP_PEER_COPY) { *why = "unknown dp_exchange"; return VB200_ERR_INVALID; }
    return VB200_OK;
}

struct PlanIdx {
    int params, grads, s1, s2, sc, mse, cs, gs, x[2], y[2], ln = -1, recv = -1;
    std::vector<int> act, pre, delta, ln_is, mask;
    int64_t ln_floats = 0;
    std::vector<int64_t> off_ln;
};

// Lay the step's buffers out on the fixed schedule (forward 0..n-1, loss n, backward
// n+1..2n, update 2n+1).  Parameters, gradients, optimizer state, scratch and the two input
// slots are persistent; activations, pre-activations and deltas are temporaries that may
// share storage when their lifetimes do not meet.
void make_plan(const vb200_config &c, ArenaPlan &pl, PlanIdx &ix, std::vector<int64_t> &off_w,
               std::vector<int64_t> &off_b, int64_t &n_weights_padded, int64_t &n_params_padded) {
    const int n = c.n_sizes - 1;
    const int *L = c.layers;
    const int B = c.batch;
    off_w.resize(n);
    off_b.resize(n);
    int64_t off = 0;
    for (int i = 0; i < n; ++i) { off_w[i] = off; off += pad64((int64_t)L[i] * L[i + 1]); }
    n_weights_padded = off;
    for (int i = 0; i < n; ++i) { off_b[i] = off; off += pad64(L[i + 1]); }
    n_params_padded = off;
    const int64_t P = off;
    const int opt = c.optimizer;
    const bool has1 = opt != VB200_OPT_SGD, has2 = (opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW);
    const int end = 2 * n + 1;
    const bool row_opts = cfg_row_opts(c), keep_pre = cfg_keep_pre(c), ln = c.use_layernorm == 1;
    const bool drop = c.dropout_p > 0.0f, clip = c.clip_grad > 0.0f;
    ix.off_ln.assign(n > 1 ? n - 1 : 0, 0);
    ix.ln_floats = 0;
    if (ln)
        for (int k = 0; k + 1 < n; ++k) { ix.off_ln[k] = ix.ln_floats; ix.ln_floats += pad64(2LL * L[k + 1]); }
    ix.params = pl.add("params", P * 4, 0, end, true);
    // gradients, then the loss slot, then the LayerNorm gradients, then the clip's norm slot
    ix.grads = pl.add("grads+loss", (P + 64 + ix.ln_floats + 64) * 4, 0, end, true);
    if (ln) ix.ln = pl.add("layernorm_params", ix.ln_floats * 4, 0, end, true);
    ix.s1 = pl.add("opt_state1", has1 ? P * 4 : 4, 0, end, true);
    ix.s2 = pl.add("opt_state2", has2 ? P * 4 : 4, 0, end, true);
    ix.sc = pl.add("scalars+status", 1024, 0, end, true);
    // exchange by copy: rank q's copy engines write its gradients (and loss sum) into slot q
    if (c.dp_exchange == VB200_DP_PEER_COPY && (c.world_size > 1 || c.force_dp == 1))
        ix.recv = pl.add("dp_receive_slots", (int64_t)(c.world_size > 1 ? c.world_size : 1) * (P + 64) * 4, 0, end, true);
    // >= one loss partial per CTA of the persistent step, and behind them its per-cluster partial outputs [<= 160][64]
    long long mse = std::max<long long>(loss_blocks((long long)B * L[n]), 256 + 64 * 160);
    if (clip) {  // block partials of every delta's sum of squares
        long long all = 0;
        for (int i = 0; i < n; ++i) all += loss_blocks((long long)B * L[i + 1]);
        mse = std::max(mse, all);
    }
    ix.mse = pl.add("mse_scratch", mse * 4, 0, end, true);
    long long cs = 0;
    for (int i = 0; i < n; ++i) {
        cs = std::max(cs, colsum_chunks(B, L[i + 1]) * (long long)L[i + 1] * ((ln && i < n - 1) ? 2 : 1));
        if (L[i + 1] == 1) cs = std::max(cs, colsum_chunks(B, L[i]) * (long long)L[i]);  // weighted sums for dW
    }
    ix.cs = pl.add("colsum_scratch", cs * 4, 0, end, true);
    long long gs = 0;  // split-K slabs of the FFMA path: the largest need over the step's GEMMs
    for (int i = 0; i < n; ++i) {
        const long long r = L[i], cc = L[i + 1];
        gs = std::max(gs, ffma_scratch_floats(B, cc, r));            // forward
        gs = std::max(gs, ffma_scratch_floats(r, cc, B));            // dW
        if (i > 0) gs = std::max(gs, ffma_scratch_floats(B, r, cc)); // dX
        // slabs of tensor GEMMs that split K to fill their last wave (not with SGD folded into dW: its
        // epilogue then runs in the slab reduction all the same, so the scratch is needed either way)
        const bool fp = c.gemm_path == VB200_GEMM_TENSOR_PAIR;
        gs = std::max(gs, gemm_tc_scratch_floats(GEMM_NN, B, cc, r, fp));
        gs = std::max(gs, gemm_tc_scratch_floats(GEMM_TN, r, cc, B, fp));
        if (i > 0) gs = std::max(gs, gemm_tc_scratch_floats(GEMM_NT, B, r, cc, fp));
    }
    ix.gs = pl.add("gemm_splitk_scratch", gs * 4, 0, end, true);
    for (int s = 0; s < 2; ++s) {
        ix.x[s] = pl.add(s ? "x_slot1" : "x_slot0", (int64_t)B * L[0] * 4, 0, end, true);
        ix.y[s] = pl.add(s ? "y_slot1" : "y_slot0", (int64_t)B * L[n] * 4, 0, end, true);
    }
    ix.act.assign(n + 1, -1);
    ix.pre.assign(n, -1);
    ix.delta.assign(n, -1);
    ix.ln_is.assign(n, -1);
    ix.mask.assign(n, -1);
    // Hidden layer k = i-1 writes act_i (and pre_k, mask_k, 1/sigma_k).  act_i is last read by dW_i;
    // with the row stages also by the backward of delta_{i-1}, one position later.  The clip moves
    // every dW behind the whole backward sweep, so activations and deltas then live to the end.
    for (int i = 1; i < n; ++i) {
        const int bwd_rows = pos_bwd(n, i - 1);
        const int act_last = clip ? end : (row_opts ? bwd_rows : pos_bwd(n, i));
        ix.act[i] = pl.add("act" + std::to_string(i), (int64_t)B * L[i] * 4, pos_fwd(i - 1), act_last, false);
        if (keep_pre)
            ix.pre[i - 1] = pl.add("pre" + std::to_string(i - 1), (int64_t)B * L[i] * 4, pos_fwd(i - 1),
                                   row_opts ? bwd_rows : pos_bwd(n, i), false);
        if (drop) ix.mask[i - 1] = pl.add("mask" + std::to_string(i - 1), (int64_t)B * L[i], pos_fwd(i - 1), bwd_rows, false);
        if (ln) ix.ln_is[i - 1] = pl.add("ln_invstd" + std::to_string(i - 1), (int64_t)B * 4, pos_fwd(i - 1), bwd_rows, false);
    }
    ix.act[n] = pl.add("act" + std::to_string(n), (int64_t)B * L[n] * 4, pos_fwd(n - 1), pos_loss(n), false);
    for (int i = n - 1; i >= 0; --i) {
        int first = (i == n - 1) ? pos_loss(n) : pos_bwd(n, i + 1);
        ix.delta[i] = pl.add("delta" + std::to_string(i), (int64_t)B * L[i + 1] * 4, first, clip ? end : pos_bwd(n, i), false);
    }
    pl.plan();
}

int build(vb200_handle *h) {
    const vb200_config &c = h->cfg;
    const int n = c.n_sizes - 1;
    h->n = n;
    h->L.assign(c.layers, c.layers + c.n_sizes);
    h->B = c.batch;
    h->world = c.world_size > 1 ? c.world_size : 1;
    h->rank = c.rank;
    const long long gb = c.global_batch ? c.global_batch : (long long)c.batch * h->world;
    h->global_nt = gb * h->L[n];
    h->use_graph = c.use_graph != 2;
    h->fuse_sgd = (c.fuse_sgd == 1) && c.optimizer == VB200_OPT_SGD && h->world == 1 && c.force_dp != 1;
    h->row_opts = cfg_row_opts(c);
    h->keep_pre = cfg_keep_pre(c);
    h->layernorm = c.use_layernorm == 1;
    h->dropout_p = c.dropout_p;
    h->clip = c.clip_grad;
    const int B = h->B;
    const std::vector<int> &L = h->L;

    PlanIdx ix;
    make_plan(c, h->plan, ix, h->off_w, h->off_b, h->n_weights_padded, h->n_params_padded);
    ArenaPlan &pl = h->plan;
    const int64_t P = h->n_params_padded;
    std::string why;
    if (!pl.verify(&why)) return h->fail(VB200_ERR_INVALID, "memory plan rejected: " + why);
    const int i_params = ix.params, i_grads = ix.grads, i_s1 = ix.s1, i_s2 = ix.s2, i_sc = ix.sc, i_mse = ix.mse,
              i_cs = ix.cs;
    const int *i_x = ix.x, *i_y = ix.y;
    const std::vector<int> &i_act = ix.act, &i_pre = ix.pre, &i_delta = ix.delta;

    // ---- one allocation
    h->arena_bytes = pl.total();
    cudaError_t e = cudaMalloc(&h->arena, (size_t)h->arena_bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        char buf[128];
        snprintf(buf, sizeof buf, "cudaMalloc of the %.2f GB arena failed: %s", h->arena_bytes / 1e9, cudaGetErrorString(e));
        return h->fail(VB200_ERR_OOM, buf);
    }
    auto at = [&](int idx) -> float * { return reinterpret_cast<float *>(h->arena + pl.offset(idx)); };
    h->params = at(i_params);
    h->grads = at(i_grads);
    h->loss_sum = h->grads + P;
    h->ln_floats = ix.ln_floats;
    h->off_ln = ix.off_ln;
    h->ln_grads = h->loss_sum + 64;
    h->clip_norm = h->ln_grads + h->ln_floats;
    if (ix.ln >= 0) h->ln_params = at(ix.ln);
    h->ln_is.assign(n, nullptr);
    h->mask.assign(n, nullptr);
    for (int k = 0; k + 1 < n; ++k) {
        if (ix.ln_is[k] >= 0) h->ln_is[k] = at(ix.ln_is[k]);
        if (ix.mask[k] >= 0) h->mask[k] = reinterpret_cast<unsigned char *>(at(ix.mask[k]));
    }
    // dropout: one draw per hidden element of the GLOBAL batch, layer after layer (:773-788); this rank's
    // rows start rank * batch rows into each layer's share
    h->draw_off.assign(n, 0);
    h->draws_per_step = 0;
    if (h->dropout_p > 0.0f)
        for (int k = 0; k + 1 < n; ++k) {
            h->draw_off[k] = h->draws_per_step + (unsigned long long)h->rank * B * L[k + 1];
            h->draws_per_step += (unsigned long long)gb * L[k + 1];
        }
    h->s1 = at(i_s1);
    h->s2 = at(i_s2);
    h->scalars = reinterpret_cast<StepScalars *>(at(i_sc));
    h->status_word = reinterpret_cast<unsigned int *>(reinterpret_cast<char *>(at(i_sc)) + 512);
    h->mse_scratch = at(i_mse);
    h->colsum_scratch = at(i_cs);
    h->gemm_scratch = at(ix.gs);
    h->gemm_scratch_floats = (long long)(pl.buffers()[(size_t)ix.gs].bytes / 4);
    h->off_params = pl.offset(i_params);
    h->off_grads = pl.offset(i_grads);
    h->off_s1 = pl.offset(i_s1);
    h->off_s2 = pl.offset(i_s2);
    h->off_flags = pl.offset(i_sc) + 768;   // 8 barrier words behind the scalars (offset 0) and the status word (512)
    h->first_bad = reinterpret_cast<unsigned long long *>(reinterpret_cast<char *>(at(i_sc)) + 832);
    h->grid_barrier = reinterpret_cast<unsigned int *>(reinterpret_cast<char *>(at(i_sc)) + 896);
    h->check_finite = c.check_finite == 1;
    {
        // limit of the data-parallel barrier waits: the configuration, else VOLTA_B200_WAIT_MS, else 4 s
        long long ms = c.device_wait_ms;
        if (ms <= 0) { const char *e = getenv("VOLTA_B200_WAIT_MS"); ms = e ? atoll(e) : 0; }
        if (ms > 0) h->wait_ns = (unsigned long long)ms * 1000000ull;
    }
    h->off_loss = h->off_grads + P * 4;
    if (ix.recv >= 0) {
        h->recv = at(ix.recv);
        h->off_recv = pl.offset(ix.recv);
        h->recv_slot_floats = P + 64;
    }

    for (int s = 0; s < 2; ++s) { h->xin[s] = at(i_x[s]); h->yin[s] = at(i_y[s]); }
    h->act.assign(n + 1, nullptr);
    h->pre.assign(n, nullptr);
    h->delta.assign(n, nullptr);
    for (int i = 1; i <= n; ++i) h->act[i] = at(i_act[i]);
    for (int i = 0; i < n; ++i) { if (i_pre[i] >= 0) h->pre[i] = at(i_pre[i]); h->delta[i] = at(i_delta[i]); }

    VB_CUDA(h, cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking));
    VB_CUDA(h, cudaStreamCreateWithFlags(&h->copy_stream, cudaStreamNonBlocking));
    for (int s = 0; s < 2; ++s) {
        VB_CUDA(h, cudaEventCreateWithFlags(&h->ev_copied[s], cudaEventDisableTiming));
        VB_CUDA(h, cudaEventCreateWithFlags(&h->ev_slot_free[s], cudaEventDisableTiming));
    }
    // zero everything persistent (the reference zero-initialises every buffer, :608-611)
    VB_CUDA(h, cudaMemsetAsync(h->arena, 0, (size_t)h->arena_bytes, h->stream));

    VB_CUDA(h, cudaMallocHost(&h->mirror_params, (size_t)P * 4));
    VB_CUDA(h, cudaMallocHost(&h->host_loss, 2 * sizeof(float)));
    VB_CUDA(h, cudaMallocHost(&h->host_status, sizeof(unsigned int)));
    VB_CUDA(h, cudaMallocHost(&h->host_first_bad, 4 * sizeof(unsigned long long)));
    for (int r = 0; r < 4; ++r) h->host_first_bad[r] = ~0ULL;
    h->host_loss[0] = h->host_loss[1] = 0.0f;
    *h->host_status = 0;
    memset(h->mirror_params, 0, (size_t)P * 4);
    uint64_t rng = 42;
    for (int i = 0; i < n; ++i)
        lcg_xavier(h->mirror_params + h->off_w[i], (int64_t)L[i] * L[i + 1], L[i], L[i + 1], &rng);
    VB_CUDA(h, cudaMemcpyAsync(h->params, h->mirror_params, (size_t)P * 4, cudaMemcpyHostToDevice, h->stream));
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    if (h->layernorm) {  // gamma = 1, beta = 0 (:660-664)
        std::vector<float> ln((size_t)h->ln_floats, 0.0f);
        for (int k = 0; k + 1 < n; ++k) std::fill_n(ln.begin() + h->off_ln[k], L[k + 1], 1.0f);
        VB_CUDA(h, cudaMemcpy(h->ln_params, ln.data(), ln.size() * 4, cudaMemcpyHostToDevice));
    }

    if (h->world > 1 || c.force_dp == 1) {
        VB_CUDA(h, cudaStreamCreateWithFlags(&h->comm_stream, cudaStreamNonBlocking));
        VB_CUDA(h, cudaEventCreateWithFlags(&h->ev_join, cudaEventDisableTiming));
        for (int q = 0; q < 2; ++q) VB_CUDA(h, cudaEventCreateWithFlags(&h->ev_clip[q], cudaEventDisableTiming));
        h->ev_bucket.resize(n + 1);
        for (auto &ev : h->ev_bucket) VB_CUDA(h, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        h->ev_dx.resize(n);
        for (auto &ev : h->ev_dx) VB_CUDA(h, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        h->dp = new DpComm();
        if (h->dp->init(c.nccl_unique_id, h->world, h->rank)) return h->fail(VB200_ERR_NCCL, h->dp->error());
        // NCCL sets up its channels and peer connections on the first collective (allocations and
        // a handshake between the ranks); that must not happen inside a stream capture.  Run one
        // plain all-reduce first (on the loss slot, which is zero here and stays zero).
        if (h->dp->all_reduce_sum(h->loss_sum, 64, h->comm_stream)) return h->fail(VB200_ERR_NCCL, h->dp->error());
        VB_CUDA(h, cudaStreamSynchronize(h->comm_stream));
    }
    // Batches of at most 64 rows on one GPU, without the optional row stages: the whole step as one
    // persistent kernel (vb_step_small.cu).  step_kernel: 0 = where it applies, 1 = never, 2 = required.
    {
        static const bool env_on = [] { const char *e = getenv("VOLTA_B200_SMALL_STEP"); return !(e && e[0] == '0'); }();
        const bool wanted = c.step_kernel == 2 || (c.step_kernel == 0 && env_on && c.gemm_path == VB200_GEMM_AUTO);
        const bool plain = h->world == 1 && c.force_dp != 1 && !h->row_opts && h->clip == 0.0f;
        if (wanted && plain && n <= kSmallStepMaxLayers) {
            int cl = 0;
            const int grid = small_step_grid(c.optimizer, &cl);
            if (grid > 0 && small_step_shape_ok(c.layers, c.n_sizes, 1, grid / cl)) {
                h->ss_grid = grid;
                h->ss_cluster = cl;
                h->ss_forward = true;
                // where it applies by default: up to 8 M parameters (VOLTA_B200_SMALL_STEP_MAX_PARAMS).  Beyond
                // that the per-kernel schedule's streaming optimizer (64 warps per SM against this kernel's 8)
                // makes up for its launches (measured on the 6.3 M-parameter configuration: 0.205 ms per step
                // here, 0.224 ms through the per-kernel schedule).
                static const long long max_params = [] { const char *e = getenv("VOLTA_B200_SMALL_STEP_MAX_PARAMS"); return e ? atoll(e) : (8LL << 20); }();
                if (B <= 64 && (c.step_kernel == 2 || h->n_params_padded <= max_params)) {
                    h->small_step = true;
                    h->fuse_sgd = false;
                }
            }
        }
        if (c.step_kernel == 2 && !h->small_step)
            return h->fail(VB200_ERR_UNSUPPORTED, "step_kernel = 2: the persistent step takes one GPU, at most 64 rows, at most 16 "
                                                  "layers of width <= 64 x (SMs / 4), and none of softmax / LayerNorm / dropout / clip");
    }
    if (h->ss_forward) {
        // one forward-only launch on a single row of the (zeroed) input slot shows whether the device takes the
        // cooperative cluster launch; if not, the per-kernel schedule serves instead
        int rc = enqueue_small_step(h, 0, 1);
        cudaError_t e = rc ? cudaErrorUnknown : cudaStreamSynchronize(h->stream);
        if (rc || e != cudaSuccess) {
            cudaGetLastError();
            if (c.step_kernel == 2) return h->fail(VB200_ERR_CUDA, "step_kernel = 2: the device refused the persistent kernel's launch: " + h->error);
            h->small_step = false;
            h->ss_forward = false;
            h->status = VB200_OK;
            h->error.clear();
        }
    }
    // Host inputs of at least 64 MB: copy and forward pass in row chunks of at least 8192 rows (the GEMMs keep
    // their efficiency at that height), so that only the first chunk's copy is exposed.  VOLTA_B200_IN_CHUNKS=1
    // switches it off, another value in 2..8 that divides the batch sets the count.
    if (!h->small_step && h->use_graph && !h->row_opts) {
        int want = 0;
        if (const char *e = getenv("VOLTA_B200_IN_CHUNKS")) want = atoi(e);
        int chunks = 1;
        if (want >= 2 && want <= vb200_handle::kMaxInChunks && B % want == 0) {
            chunks = want;
        } else if (want == 0 && (long long)B * L[0] * 4 >= (64LL << 20)) {
            for (int cnum = vb200_handle::kMaxInChunks; cnum >= 2; cnum /= 2)
                if (B % cnum == 0 && B / cnum >= 8192) { chunks = cnum; break; }
        }
        h->in_chunks = chunks;
        if (chunks > 1)
            for (int sl = 0; sl < 2; ++sl)
                for (int cc = 0; cc < chunks; ++cc) VB_CUDA(h, cudaEventCreateWithFlags(&h->ev_chunk[sl][cc], cudaEventDisableTiming));
    }
    if (h->small_step) {
        h->kernels_per_step = 1;   // launched directly every step, with the step's scalars as an argument
    } else if (h->use_graph) {
        int rc = capture_graphs(h);
        if (rc) return rc;
    } else {
        // count the launches of one step without running it: the schedule is fixed
        h->kernels_per_step = 0;
    }
    return VB200_OK;
}

}  // namespace

// =========================================================================================
// C ABI
// =========================================================================================
extern "C" {

const char *volta_b200_version(void) { return "volta_b200 0.1 (sm_100a)"; }
int32_t volta_b200_config_size(void) { return (int32_t)sizeof(vb200_config); }

int volta_b200_create(const vb200_config *cfg, vb200_handle **out) {
    if (out) *out = nullptr;
    std::string why;
    int rc = validate(cfg, &why);
    if (!out && rc == VB200_OK) { rc = VB200_ERR_INVALID; why = "null output pointer"; }
    if (rc == VB200_OK) {
        int ndev = 0;
        cudaError_t e = cudaGetDeviceCount(&ndev);
        if (e != cudaSuccess || ndev == 0) {
            cudaGetLastError();
            rc = VB200_ERR_CUDA;
            why = "no CUDA device available: libvolta_b200 has no CPU fallback";
        }
    }
    if (rc != VB200_OK) {
        std::lock_guard<std::mutex> lk(g_err_mutex);
        g_create_status = rc;
        g_create_error = why;
        return rc;
    }
    vb200_handle *h = new vb200_handle();
    h->cfg = *cfg;
    rc = build(h);
    if (rc != VB200_OK) {
        {
            std::lock_guard<std::mutex> lk(g_err_mutex);
            g_create_status = rc;
            g_create_error = h->error;
        }
        destroy(h);
        return rc;
    }
    *out = h;
    return VB200_OK;
}

void volta_b200_destroy(vb200_handle *h) { destroy(h); }

int volta_b200_step(vb200_handle *h, const float *X, const float *Y, float lr) {
    if (!h) return VB200_ERR_INVALID;
    return do_step(h, X, Y, lr, false);
}

float volta_b200_loss(vb200_handle *h) {
    if (!h) return NAN;
    if (cudaStreamSynchronize(h->stream) != cudaSuccess) {
        h->fail(VB200_ERR_CUDA, std::string("stream failed: ") + cudaGetErrorString(cudaGetLastError()));
        return NAN;
    }
    check_device_status(h);
    // mlp_train_rust_codegen.rs:798: last_loss = lacc / nt
    return h->host_loss[h->last_slot] / (float)h->global_nt;
}

int volta_b200_set_params(vb200_handle *h, int32_t li, const float *w, const float *b) {
    if (!h) return VB200_ERR_INVALID;
    if (li < 0 || li >= h->n) return VB200_OK;  // ignored, as in the reference
    if (!w || !b) return h->reject(VB200_ERR_INVALID, "set_params: null pointer");
    const size_t wn = (size_t)h->L[li] * h->L[li + 1], bn = (size_t)h->L[li + 1];
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    // w and b may be host or device pointers (unified addressing tells which)
    VB_CUDA(h, cudaMemcpy(h->params + h->off_w[li], w, wn * 4, cudaMemcpyDefault));
    VB_CUDA(h, cudaMemcpy(h->params + h->off_b[li], b, bn * 4, cudaMemcpyDefault));
    return VB200_OK;
}

int volta_b200_get_params(vb200_handle *h, float **wo, float **bo) {
    if (!h || !wo || !bo) return VB200_ERR_INVALID;
    VB_CUDA(h, cudaMemcpyAsync(h->mirror_params, h->params, (size_t)h->n_params_padded * 4, cudaMemcpyDeviceToHost,
                               h->stream));
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    for (int i = 0; i < h->n; ++i) {
        wo[i] = h->mirror_params + h->off_w[i];
        bo[i] = h->mirror_params + h->off_b[i];
    }
    return check_device_status(h);
}

int volta_b200_get_grads(vb200_handle *h, float **dwo, float **dbo) {
    if (!h || !dwo || !dbo) return VB200_ERR_INVALID;
    if (!h->mirror_grads) VB_CUDA(h, cudaMallocHost(&h->mirror_grads, (size_t)h->n_params_padded * 4));
    VB_CUDA(h, cudaMemcpyAsync(h->mirror_grads, h->grads, (size_t)h->n_params_padded * 4, cudaMemcpyDeviceToHost,
                               h->stream));
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    for (int i = 0; i < h->n; ++i) {
        dwo[i] = h->mirror_grads + h->off_w[i];
        dbo[i] = h->mirror_grads + h->off_b[i];
    }
    return VB200_OK;
}

namespace {
int64_t moment_floats(vb200_handle *h) {
    const int opt = h->cfg.optimizer;
    if (opt == VB200_OPT_SGD) return 0;
    return (opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW) ? 2 * h->n_params_padded : h->n_params_padded;
}
}  // namespace

int64_t volta_b200_state_floats(vb200_handle *h) {
    if (!h) return 0;
    return moment_floats(h) + (h->dropout_p > 0.0f ? 2 : 0);
}

int volta_b200_get_layernorm(vb200_handle *h, int32_t li, float *gamma, float *beta) {
    if (!h) return VB200_ERR_INVALID;
    if (!h->layernorm) return h->reject(VB200_ERR_INVALID, "get_layernorm: the handle was created without LayerNorm");
    if (li < 0 || li >= h->n - 1 || !gamma || !beta) return h->reject(VB200_ERR_INVALID, "get_layernorm: bad layer index or null pointer");
    const size_t c = (size_t)h->L[li + 1];
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    VB_CUDA(h, cudaMemcpy(gamma, h->ln_params + h->off_ln[li], c * 4, cudaMemcpyDeviceToHost));
    VB_CUDA(h, cudaMemcpy(beta, h->ln_params + h->off_ln[li] + c, c * 4, cudaMemcpyDeviceToHost));
    return check_device_status(h);
}

int volta_b200_set_layernorm(vb200_handle *h, int32_t li, const float *gamma, const float *beta) {
    if (!h) return VB200_ERR_INVALID;
    if (!h->layernorm) return h->reject(VB200_ERR_INVALID, "set_layernorm: the handle was created without LayerNorm");
    if (li < 0 || li >= h->n - 1 || !gamma || !beta) return h->reject(VB200_ERR_INVALID, "set_layernorm: bad layer index or null pointer");
    const size_t c = (size_t)h->L[li + 1];
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    VB_CUDA(h, cudaMemcpy(h->ln_params + h->off_ln[li], gamma, c * 4, cudaMemcpyHostToDevice));
    VB_CUDA(h, cudaMemcpy(h->ln_params + h->off_ln[li] + c, beta, c * 4, cudaMemcpyHostToDevice));
    return VB200_OK;
}

int volta_b200_save_state(vb200_handle *h, float *out, int64_t n, uint64_t *step_out) {
    if (!h) return VB200_ERR_INVALID;
    if (h->dp_fused) return h->reject(VB200_ERR_UNSUPPORTED, "save_state: optimizer state is sharded over the ranks in fused data-parallel mode");
    const int64_t need = volta_b200_state_floats(h), mom = moment_floats(h);
    if (n < need || (need && !out)) return h->reject(VB200_ERR_INVALID, "save_state: buffer too small");
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    const int64_t P = h->n_params_padded;
    if (mom >= P) VB_CUDA(h, cudaMemcpy(out, h->s1, (size_t)P * 4, cudaMemcpyDeviceToHost));
    if (mom >= 2 * P) VB_CUDA(h, cudaMemcpy(out + P, h->s2, (size_t)P * 4, cudaMemcpyDeviceToHost));
    if (need > mom) memcpy(out + mom, &h->dropout_rng, 8);  // raw bits of the mask stream position
    if (step_out) *step_out = h->adam_step;
    return VB200_OK;
}

int volta_b200_load_state(vb200_handle *h, const float *in, int64_t n, uint64_t step) {
    if (!h) return VB200_ERR_INVALID;
    const int64_t need = volta_b200_state_floats(h), mom = moment_floats(h);
    if (n < need || (need && !in)) return h->reject(VB200_ERR_INVALID, "load_state: buffer too small");
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    const int64_t P = h->n_params_padded;
    if (mom >= P) VB_CUDA(h, cudaMemcpy(h->s1, in, (size_t)P * 4, cudaMemcpyHostToDevice));
    if (mom >= 2 * P) VB_CUDA(h, cudaMemcpy(h->s2, in + P, (size_t)P * 4, cudaMemcpyHostToDevice));
    if (need > mom) memcpy(&h->dropout_rng, in + mom, 8);
    h->adam_step = step;
    return VB200_OK;
}

// ---- checkpoints ------------------------------------------------------------------------------
struct vb200_checkpoint {
    vb::Checkpoint ck;
};

namespace {
void set_global_error(int code, const std::string &msg) {
    std::lock_guard<std::mutex> lk(g_err_mutex);
    g_create_status = code;
    g_create_error = msg;
}
const char *state1_suffix(int opt) {
    switch (opt) {
    case VB200_OPT_ADAM:
    case VB200_OPT_ADAMW: return ".m";
    case VB200_OPT_ADAGRAD: return ".acc";
    case VB200_OPT_SGD_MOMENTUM: return ".mom";
    }
    return nullptr;
}

// Which checkpoint entries feed layer i: "<base[i]>.weight" [in, out] and "<base[i]>.bias" [out].
// The reference names a layer's tensors after the layer's user-chosen name
// (src/engine/model/layers.rs:52-58: "{name}.weight", "{name}.bias"), so the bases are
//   1. the caller's names, where given (a null entry stands for "layer<i>");
//   2. else "layer<i>", the names this library writes, if the checkpoint holds any of them;
//   3. else the prefixes X of all entries "X.weight" (2-D) that have an "X.bias", in the sorted order
//      the reference's writer uses, provided there are exactly n of them and their shapes are the
//      topology's, layer by layer.
// Returns how many parameter tensors (weights and biases) were found with the right shape; 0 or a
// wrong shape fills *why.
int resolve_layer_names(const std::vector<int> &L, const vb::Checkpoint &ck, const char *const *names, int32_t n_names,
                        std::vector<std::string> *base, std::string *why) {
    const int n = (int)L.size() - 1;
    base->assign((size_t)n, std::string());
    auto count_matches = [&](bool *bad_shape) -> int {
        int found = 0;
        for (int i = 0; i < n; ++i) {
            const int64_t r = L[(size_t)i], c = L[(size_t)i + 1];
            if (const vb::CheckpointEntry *e = ck.find((*base)[(size_t)i] + ".weight")) {
                if (e->shape != std::vector<int64_t>{r, c}) { *bad_shape = true; *why = "'" + e->name + "' has the wrong shape"; return 0; }
                ++found;
            }
            if (const vb::CheckpointEntry *e = ck.find((*base)[(size_t)i] + ".bias")) {
                if (e->shape != std::vector<int64_t>{c}) { *bad_shape = true; *why = "'" + e->name + "' has the wrong shape"; return 0; }
                ++found;
            }
        }
        return found;
    };
    bool bad = false;
    if (names) {
        if (n_names != n) { *why = "need one layer name per weight layer"; return 0; }
        for (int i = 0; i < n; ++i) (*base)[(size_t)i] = names[i] ? std::string(names[i]) : "layer" + std::to_string(i);
        const int found = count_matches(&bad);
        if (!found && !bad) *why = "the checkpoint holds no '<name>.weight' or '<name>.bias' for the given layer names";
        return found;
    }
    for (int i = 0; i < n; ++i) (*base)[(size_t)i] = "layer" + std::to_string(i);
    int found = count_matches(&bad);
    if (found || bad) return found;
    std::vector<std::string> prefixes;
    for (const vb::CheckpointEntry &e : ck.entries) {
        const std::string sfx = ".weight";
        if (e.name.size() > sfx.size() && e.name.compare(e.name.size() - sfx.size(), sfx.size(), sfx) == 0 &&
            e.shape.size() == 2) {
            const std::string p = e.name.substr(0, e.name.size() - sfx.size());
            if (ck.find(p + ".bias")) prefixes.push_back(p);
        }
    }
    std::sort(prefixes.begin(), prefixes.end());
    if ((int)prefixes.size() != n) {
        *why = "no tensor is named 'layer<i>.weight' / 'layer<i>.bias', and the checkpoint's " +
               std::to_string(prefixes.size()) + " '<name>.weight' + '<name>.bias' pairs do not number the topology's " +
               std::to_string(n) + " layers: pass the layer names";
        return 0;
    }
    *base = prefixes;
    found = count_matches(&bad);
    if (bad) *why += " (layers taken in sorted name order; pass the layer names to choose another order)";
    return found;
}
}  // namespace

vb200_checkpoint *volta_b200_checkpoint_new(void) { return new vb200_checkpoint(); }

void volta_b200_checkpoint_free(vb200_checkpoint *ck) { delete ck; }

int volta_b200_checkpoint_add(vb200_checkpoint *ck, const char *name, const int64_t *shape, int32_t ndim, const float *data) {
    if (!ck || !name || ndim < 0 || (ndim && !shape)) return VB200_ERR_INVALID;
    std::vector<int64_t> sh(shape, shape + ndim);
    size_t count = 1;
    for (int64_t d : sh) {
        if (d < 0) return VB200_ERR_INVALID;
        count *= (size_t)d;
    }
    if (count && !data) return VB200_ERR_INVALID;
    ck->ck.put(name, sh, data, count);
    return VB200_OK;
}

int volta_b200_checkpoint_save(const vb200_checkpoint *ck, const char *path, int32_t format) {
    if (!ck || !path) return VB200_ERR_INVALID;
    std::string err;
    if (!vb::checkpoint_save(ck->ck, path, format, &err)) {
        set_global_error(VB200_ERR_INVALID, err);
        return VB200_ERR_INVALID;
    }
    return VB200_OK;
}

vb200_checkpoint *volta_b200_checkpoint_load(const char *path) {
    if (!path) return nullptr;
    vb200_checkpoint *ck = new vb200_checkpoint();
    std::string err;
    if (!vb::checkpoint_load(&ck->ck, path, &err)) {
        set_global_error(VB200_ERR_INVALID, err);
        delete ck;
        return nullptr;
    }
    return ck;
}

vb200_checkpoint *volta_b200_checkpoint_parse(const void *bytes, int64_t n) {
    if (!bytes || n < 0) return nullptr;
    vb200_checkpoint *ck = new vb200_checkpoint();
    std::string err;
    if (!vb::checkpoint_parse(&ck->ck, std::string(static_cast<const char *>(bytes), (size_t)n), &err)) {
        set_global_error(VB200_ERR_INVALID, err);
        delete ck;
        return nullptr;
    }
    return ck;
}

int32_t volta_b200_checkpoint_count(const vb200_checkpoint *ck) { return ck ? (int32_t)ck->ck.entries.size() : 0; }

int volta_b200_checkpoint_entry(const vb200_checkpoint *ck, int32_t i, const char **name, const int64_t **shape,
                                int32_t *ndim, const float **data, int64_t *count) {
    if (!ck || i < 0 || i >= (int32_t)ck->ck.entries.size()) return VB200_ERR_INVALID;
    const vb::CheckpointEntry &e = ck->ck.entries[(size_t)i];
    if (name) *name = e.name.c_str();
    if (shape) *shape = e.shape.data();
    if (ndim) *ndim = (int32_t)e.shape.size();
    if (data) *data = e.data.data();
    if (count) *count = (int64_t)e.data.size();
    return VB200_OK;
}

int volta_b200_checkpoint_match(const vb200_config *cfg, const vb200_checkpoint *ck, const char *const *layer_names,
                                int32_t n_names) {
    std::string why;
    int rc = validate(cfg, &why);
    if (rc == VB200_OK && !ck) { rc = VB200_ERR_INVALID; why = "null checkpoint"; }
    if (rc != VB200_OK) {
        set_global_error(rc, why);
        return -rc;
    }
    std::vector<std::string> base;
    const int found = resolve_layer_names(std::vector<int>(cfg->layers, cfg->layers + cfg->n_sizes), ck->ck, layer_names,
                                          n_names, &base, &why);
    if (!found) {
        set_global_error(VB200_ERR_INVALID, why);
        return -VB200_ERR_INVALID;
    }
    return found;
}

int volta_b200_export_checkpoint(vb200_handle *h, vb200_checkpoint *ck, int32_t with_state) {
    return volta_b200_export_checkpoint_named(h, ck, with_state, nullptr, 0);
}

int volta_b200_export_checkpoint_named(vb200_handle *h, vb200_checkpoint *ck, int32_t with_state,
                                       const char *const *layer_names, int32_t n_names) {
    if (!h || !ck) return VB200_ERR_INVALID;
    if (layer_names && n_names != h->n) return h->reject(VB200_ERR_INVALID, "export_checkpoint: need one layer name per weight layer");
    auto base_of = [&](int i) -> std::string {
        return (layer_names && layer_names[i]) ? std::string(layer_names[i]) : "layer" + std::to_string(i);
    };
    if (with_state && h->dp_fused)
        return h->reject(VB200_ERR_UNSUPPORTED, "export_checkpoint: optimizer state is sharded over the ranks in fused data-parallel mode");
    const int opt = h->cfg.optimizer;
    const int64_t P = h->n_params_padded;
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    std::vector<float> host((size_t)P);
    auto put_flat = [&](const float *dev, const char *wsuffix, const char *bsuffix) -> int {
        VB_CUDA(h, cudaMemcpy(host.data(), dev, (size_t)P * 4, cudaMemcpyDeviceToHost));
        for (int i = 0; i < h->n; ++i) {
            const int64_t r = h->L[i], c = h->L[i + 1];
            const std::string base = base_of(i);
            ck->ck.put(base + wsuffix, {r, c}, host.data() + h->off_w[i], (size_t)(r * c));
            ck->ck.put(base + bsuffix, {c}, host.data() + h->off_b[i], (size_t)c);
        }
        return VB200_OK;
    };
    int rc = put_flat(h->params, ".weight", ".bias");
    if (rc) return rc;
    if (h->layernorm) {
        std::vector<float> ln((size_t)h->ln_floats);
        VB_CUDA(h, cudaMemcpy(ln.data(), h->ln_params, ln.size() * 4, cudaMemcpyDeviceToHost));
        for (int k = 0; k + 1 < h->n; ++k) {
            const int64_t c = h->L[k + 1];
            ck->ck.put(base_of(k) + ".ln_gamma", {c}, ln.data() + h->off_ln[k], (size_t)c);
            ck->ck.put(base_of(k) + ".ln_beta", {c}, ln.data() + h->off_ln[k] + c, (size_t)c);
        }
    }
    if (with_state) {
        if (const char *sfx = state1_suffix(opt)) {
            const std::string ws = std::string(".weight") + sfx, bs = std::string(".bias") + sfx;
            rc = put_flat(h->s1, ws.c_str(), bs.c_str());
            if (rc) return rc;
        }
        if (opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW) {
            rc = put_flat(h->s2, ".weight.v", ".bias.v");
            if (rc) return rc;
            float parts[3];
            vb::split_u64(h->adam_step, parts);
            ck->ck.put("meta.adam_step", {3}, parts, 3);
        }
        if (h->dropout_p > 0.0f) {
            float parts[3];
            vb::split_u64(h->dropout_rng, parts);
            ck->ck.put("meta.dropout_rng", {3}, parts, 3);
        }
    }
    return check_device_status(h);
}

int volta_b200_import_checkpoint(vb200_handle *h, const vb200_checkpoint *ck) {
    return volta_b200_import_checkpoint_named(h, ck, nullptr, 0);
}

int volta_b200_import_checkpoint_named(vb200_handle *h, const vb200_checkpoint *ck, const char *const *layer_names,
                                       int32_t n_names) {
    if (!h || !ck) return VB200_ERR_INVALID;
    std::vector<std::string> bases;
    {
        // a checkpoint that names none of this topology's parameters is an error, not a silent no-op
        std::string why;
        if (!resolve_layer_names(h->L, ck->ck, layer_names, n_names, &bases, &why))
            return h->reject(VB200_ERR_INVALID, "import_checkpoint: " + why);
    }
    const int opt = h->cfg.optimizer;
    const int64_t P = h->n_params_padded;
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    std::vector<float> host((size_t)P);
    // every tensor of the flat region that the checkpoint names replaces the handle's; the rest stays
    auto take_flat = [&](float *dev, const std::string &wsuffix, const std::string &bsuffix) -> int {
        VB_CUDA(h, cudaMemcpy(host.data(), dev, (size_t)P * 4, cudaMemcpyDeviceToHost));
        bool any = false;
        for (int i = 0; i < h->n; ++i) {
            const int64_t r = h->L[i], c = h->L[i + 1];
            const std::string &base = bases[(size_t)i];
            if (const vb::CheckpointEntry *e = ck->ck.find(base + wsuffix)) {
                if (e->shape != std::vector<int64_t>{r, c})
                    return h->reject(VB200_ERR_INVALID, "import_checkpoint: '" + e->name + "' has the wrong shape");
                memcpy(host.data() + h->off_w[i], e->data.data(), (size_t)(r * c) * 4);
                any = true;
            }
            if (const vb::CheckpointEntry *e = ck->ck.find(base + bsuffix)) {
                if (e->shape != std::vector<int64_t>{c})
                    return h->reject(VB200_ERR_INVALID, "import_checkpoint: '" + e->name + "' has the wrong shape");
                memcpy(host.data() + h->off_b[i], e->data.data(), (size_t)c * 4);
                any = true;
            }
        }
        if (any) VB_CUDA(h, cudaMemcpy(dev, host.data(), (size_t)P * 4, cudaMemcpyHostToDevice));
        return VB200_OK;
    };
    int rc = take_flat(h->params, ".weight", ".bias");
    if (rc) return rc;
    if (h->layernorm) {
        std::vector<float> ln((size_t)h->ln_floats);
        VB_CUDA(h, cudaMemcpy(ln.data(), h->ln_params, ln.size() * 4, cudaMemcpyDeviceToHost));
        for (int k = 0; k + 1 < h->n; ++k) {
            const int64_t c = h->L[k + 1];
            const vb::CheckpointEntry *g = ck->ck.find(bases[(size_t)k] + ".ln_gamma");
            const vb::CheckpointEntry *b = ck->ck.find(bases[(size_t)k] + ".ln_beta");
            for (const vb::CheckpointEntry *e : {g, b})
                if (e && e->shape != std::vector<int64_t>{c})
                    return h->reject(VB200_ERR_INVALID, "import_checkpoint: '" + e->name + "' has the wrong shape");
            if (g) memcpy(ln.data() + h->off_ln[k], g->data.data(), (size_t)c * 4);
            if (b) memcpy(ln.data() + h->off_ln[k] + c, b->data.data(), (size_t)c * 4);
        }
        VB_CUDA(h, cudaMemcpy(h->ln_params, ln.data(), ln.size() * 4, cudaMemcpyHostToDevice));
    }
    if (h->dp_fused) return VB200_OK;  // sharded state: parameters only
    if (const char *sfx = state1_suffix(opt)) {
        rc = take_flat(h->s1, std::string(".weight") + sfx, std::string(".bias") + sfx);
        if (rc) return rc;
    }
    if (opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW) {
        rc = take_flat(h->s2, ".weight.v", ".bias.v");
        if (rc) return rc;
        if (const vb::CheckpointEntry *e = ck->ck.find("meta.adam_step")) {
            uint64_t v = 0;
            if (e->data.size() != 3 || !vb::join_u64(e->data.data(), &v))
                return h->reject(VB200_ERR_INVALID, "import_checkpoint: 'meta.adam_step' is not a split counter");
            h->adam_step = v;
        }
    }
    if (h->dropout_p > 0.0f)
        if (const vb::CheckpointEntry *e = ck->ck.find("meta.dropout_rng")) {
            uint64_t v = 0;
            if (e->data.size() != 3 || !vb::join_u64(e->data.data(), &v))
                return h->reject(VB200_ERR_INVALID, "import_checkpoint: 'meta.dropout_rng' is not a split counter");
            h->dropout_rng = v;
        }
    return VB200_OK;
}

int volta_b200_status(vb200_handle *h) {
    if (!h) {
        std::lock_guard<std::mutex> lk(g_err_mutex);
        return g_create_status;
    }
    return h->status;
}

const char *volta_b200_last_error(vb200_handle *h) {
    if (!h) {
        std::lock_guard<std::mutex> lk(g_err_mutex);
        return g_create_error.c_str();
    }
    return h->error.c_str();
}

void *volta_b200_stream(vb200_handle *h) { return h ? (void *)h->stream : nullptr; }

int volta_b200_synchronize(vb200_handle *h) {
    if (!h) return VB200_ERR_INVALID;
    VB_CUDA(h, cudaStreamSynchronize(h->copy_stream));
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    return check_device_status(h);
}

int64_t volta_b200_arena_bytes(vb200_handle *h) { return h ? h->arena_bytes : 0; }

int volta_b200_plan(const vb200_config *cfg, int64_t *arena_bytes, int64_t *unshared_bytes, char *report,
                    int64_t report_len) {
    std::string why;
    int rc = validate(cfg, &why);
    if (rc) {
        std::lock_guard<std::mutex> lk(g_err_mutex);
        g_create_status = rc;
        g_create_error = why;
        return rc;
    }
    ArenaPlan pl;
    PlanIdx ix;
    std::vector<int64_t> ow, ob;
    int64_t nw = 0, np = 0;
    make_plan(*cfg, pl, ix, ow, ob, nw, np);
    if (!pl.verify(&why)) {
        std::lock_guard<std::mutex> lk(g_err_mutex);
        g_create_status = VB200_ERR_INVALID;
        g_create_error = "memory plan rejected: " + why;
        return VB200_ERR_INVALID;
    }
    if (arena_bytes) *arena_bytes = pl.total();
    if (unshared_bytes) *unshared_bytes = pl.sum_unshared();
    if (report && report_len > 0) {
        std::string txt;
        char line[160];
        for (auto &b : pl.buffers()) {
            snprintf(line, sizeof line, "%s %lld %lld %d %d %d\n", b.name.c_str(), (long long)b.offset,
                     (long long)b.bytes, b.first_use, b.last_use, b.persistent ? 1 : 0);
            txt += line;
        }
        strncpy(report, txt.c_str(), (size_t)report_len - 1);
        report[report_len - 1] = 0;
    }
    return VB200_OK;
}
int32_t volta_b200_kernels_per_step(vb200_handle *h) { return h ? h->kernels_per_step : 0; }

int volta_b200_profile_step(vb200_handle *h, const float *X, const float *Y, float lr, vb200_kernel_record *out,
                            int32_t max) {
    if (!h) return -VB200_ERR_INVALID;
    if (h->dp_fused) return -h->reject(VB200_ERR_UNSUPPORTED, "profile_step: not with the fused peer-memory exchange");
    for (auto &r : h->records) { cudaEventDestroy(r.e0); cudaEventDestroy(r.e1); }
    h->records.clear();
    int rc = do_step(h, X, Y, lr, true);
    if (rc) return -rc;
    if (cudaStreamSynchronize(h->stream) != cudaSuccess) {
        h->fail(VB200_ERR_CUDA, "profile_step: stream failed");
        return -VB200_ERR_CUDA;
    }
    int cnt = 0;
    for (auto &r : h->records) {
        if (cnt >= max || !out) break;
        vb200_kernel_record &o = out[cnt++];
        memset(&o, 0, sizeof o);
        strncpy(o.name, r.name.c_str(), sizeof(o.name) - 1);
        cudaEventElapsedTime(&o.ms, r.e0, r.e1);
        o.flops = r.flops;
        o.bytes = r.bytes;
    }
    return cnt;
}

int volta_b200_infer(vb200_handle *h, const float *in, int64_t in_n, float *out, int64_t out_n) {
    if (!h) return VB200_ERR_INVALID;
    if (!in || !out) return h->reject(VB200_ERR_INVALID, "infer: null pointer");
    const int64_t L0 = h->L[0], Ln = h->L[h->n];
    if (in_n <= 0 || in_n % L0 != 0) return h->reject(VB200_ERR_INVALID, "infer: input length is not a multiple of the input width");
    const int64_t rows = in_n / L0;
    if (rows > h->B) return h->reject(VB200_ERR_INVALID, "infer: more rows than the handle's batch");
    if (out_n != rows * Ln) return h->reject(VB200_ERR_INVALID, "infer: output length does not match rows x output width");
    // between steps only: wait for queued training work, then reuse its buffers
    VB_CUDA(h, cudaStreamSynchronize(h->copy_stream));
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    cudaPointerAttributes ai{}, ao{};
    bool idev = false, odev = false;
    if (cudaPointerGetAttributes(&ai, in) == cudaSuccess) idev = ai.type == cudaMemoryTypeDevice || ai.type == cudaMemoryTypeManaged; else cudaGetLastError();
    if (cudaPointerGetAttributes(&ao, out) == cudaSuccess) odev = ao.type == cudaMemoryTypeDevice || ao.type == cudaMemoryTypeManaged; else cudaGetLastError();
    const size_t in_bytes = (size_t)in_n * 4, out_bytes = (size_t)out_n * 4;
    // Host callers of small batches (the reference's protocol: 10 000 calls of one row, 1 000 of 64;
    // examples/bench_infer.c) are bound by launch and copy latency: stage through pinned memory and
    // replay ONE captured graph per row count (copy in, every layer, copy out).
    const bool staged = !idev && !odev && in_bytes <= (8u << 20) && out_bytes <= (8u << 20) && h->use_graph;
    if (staged) {
        if (!h->infer_in) {
            const size_t cap_in = std::min<size_t>((size_t)h->B * L0 * 4, 8u << 20);
            const size_t cap_out = std::min<size_t>((size_t)h->B * Ln * 4, 8u << 20);
            VB_CUDA(h, cudaMallocHost(&h->infer_in, cap_in));
            VB_CUDA(h, cudaMallocHost(&h->infer_out, cap_out));
        }
        auto it = h->infer_graphs.find(rows);
        if (it == h->infer_graphs.end() && h->infer_graphs.size() < 16) {
            cudaGraph_t g = nullptr;
            const int saved = h->kernels_per_step;
            VB_CUDA(h, cudaStreamBeginCapture(h->stream, cudaStreamCaptureModeThreadLocal));
            // A few rows: the first layer reads the pinned input and the last one writes the pinned output
            // directly (both are mapped into the device's address space), which saves the two copy nodes.
            // Only when both layers take kernels that use plain loads and stores (never a TMA descriptor
            // over host memory): the small-row kernel, or the row-dot of a width-one output.
            const int nl = h->n;
            const bool first_ok = h->cfg.gemm_path == VB200_GEMM_AUTO &&
                                  gemv_rows_supported(h->params + h->off_w[0], rows, h->L[1], h->L[0]);
            const bool last_ok = h->L[nl] == 1 || (h->cfg.gemm_path == VB200_GEMM_AUTO &&
                                                   gemv_rows_supported(h->params + h->off_w[nl - 1], rows, h->L[nl], h->L[nl - 1]));
            const bool direct = rows <= 8 && nl >= 2 && first_ok && last_ok;
            cudaError_t e1 = direct ? cudaSuccess
                                    : cudaMemcpyAsync(h->xin[0], h->infer_in, in_bytes, cudaMemcpyHostToDevice, h->stream);
            int rc = e1 != cudaSuccess ? VB200_ERR_CUDA
                     : direct          ? enqueue_forward(h, 0, rows, false, h->infer_in, h->infer_out)
                                       : enqueue_forward(h, 0, rows, false);
            cudaError_t e2 = direct ? cudaSuccess
                                    : cudaMemcpyAsync(h->infer_out, h->act[h->n], out_bytes, cudaMemcpyDeviceToHost, h->stream);
            cudaError_t e3 = cudaStreamEndCapture(h->stream, &g);
            h->kernels_per_step = saved;
            if (rc || e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess) {
                if (g) cudaGraphDestroy(g);
                cudaGetLastError();
                return rc ? rc : h->fail(VB200_ERR_CUDA, "infer: capturing the forward graph failed");
            }
            cudaGraphExec_t ge = nullptr;
            cudaError_t e4 = cudaGraphInstantiate(&ge, g, 0);
            cudaGraphDestroy(g);
            if (e4 != cudaSuccess) return h->fail(VB200_ERR_CUDA, std::string("infer: cudaGraphInstantiate: ") + cudaGetErrorString(e4));
            it = h->infer_graphs.emplace(rows, ge).first;
        }
        if (it != h->infer_graphs.end()) {
            memcpy(h->infer_in, in, in_bytes);
            VB_CUDA(h, cudaGraphLaunch(it->second, h->stream));
            VB_CUDA(h, cudaStreamSynchronize(h->stream));
            memcpy(out, h->infer_out, out_bytes);
            return VB200_OK;
        }
    }
    VB_CUDA(h, cudaMemcpyAsync(h->xin[0], in, in_bytes, idev ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, h->stream));
    const int saved = h->kernels_per_step;
    int rc = enqueue_forward(h, 0, rows, false);
    h->kernels_per_step = saved;
    if (rc) return rc;
    VB_CUDA(h, cudaMemcpyAsync(out, h->act[h->n], out_bytes, odev ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, h->stream));
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    return check_device_status(h);
}

int volta_b200_dp_ipc_handle(vb200_handle *h, uint8_t out[64]) {
    if (!h || !out) return VB200_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t ipc;
    VB_CUDA(h, cudaIpcGetMemHandle(&ipc, h->arena));
    memcpy(out, &ipc, 64);
    return VB200_OK;
}

int volta_b200_dp_attach_peers(vb200_handle *h, const uint8_t *handles, int32_t count) {
    if (!h) return VB200_ERR_INVALID;
    if (!h->dp) return h->reject(VB200_ERR_INVALID, "attach_peers: the handle was not created for data parallelism");
    if (count != h->world || count > kMaxPeers || !handles)
        return h->reject(VB200_ERR_INVALID, "attach_peers: need one 64-byte handle per rank (at most 8 ranks)");
    if (h->dp_fused || h->dp_copy) return h->reject(VB200_ERR_INVALID, "attach_peers: already attached");
    const bool by_copy = h->cfg.dp_exchange == VB200_DP_PEER_COPY;
    if (by_copy && !h->recv) return h->reject(VB200_ERR_INVALID, "attach_peers: the handle has no receive slots");
    if (h->layernorm || h->clip > 0.0f)
        return h->reject(VB200_ERR_UNSUPPORTED, "attach_peers: LayerNorm and the clip need the NCCL data-parallel path");
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    for (int q = 0; q < count; ++q) {
        if (q == h->rank) {
            h->peers.base[q] = h->arena;
            continue;
        }
        cudaIpcMemHandle_t ipc;
        memcpy(&ipc, handles + 64 * q, 64);
        void *p = nullptr;
        VB_CUDA(h, cudaIpcOpenMemHandle(&p, ipc, cudaIpcMemLazyEnablePeerAccess));
        h->peer_mappings.push_back(p);
        h->peers.base[q] = static_cast<char *>(p);
    }
    // from now on the step graph uses the peer-memory buckets instead of NCCL + the flat optimizer
    destroy_step_graphs(h);
    (by_copy ? h->dp_copy : h->dp_fused) = true;
    if (h->use_graph) {
        int rc = capture_graphs(h);
        if (rc) return rc;
    }
    return VB200_OK;
}

int volta_b200_dp_wait_selftest(vb200_handle *h, int32_t declared_world, int32_t wait_ms) {
    if (!h) return VB200_ERR_INVALID;
    if (declared_world < 2 || declared_world > kMaxPeers || wait_ms <= 0 || wait_ms > 10000)
        return h->reject(VB200_ERR_INVALID, "dp_wait_selftest: world must lie in 2..8 and wait_ms in 1..10000");
    if (h->dp_fused || h->dp_copy) return h->reject(VB200_ERR_INVALID, "dp_wait_selftest: not on a handle attached to peers");
    // every "peer" is this handle's own arena: slot 0 of the flag words gets written, the others never do
    PeerTable self{};
    for (int q = 0; q < kMaxPeers; ++q) self.base[q] = h->arena;
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    VB_CUDA(h, launch_dp_barrier(self, h->off_flags, declared_world, 0, h->scalars, 1u, 0x7ffffff0u, h->status_word,
                                 (unsigned long long)wait_ms * 1000000ull, h->stream));
    VB_CUDA(h, cudaMemcpyAsync(h->host_status, h->status_word, sizeof(unsigned int), cudaMemcpyDeviceToHost, h->stream));
    VB_CUDA(h, cudaStreamSynchronize(h->stream));
    return check_device_status(h);
}

int volta_b200_dp_unique_id(uint8_t out[128]) {
    if (!out) return VB200_ERR_INVALID;
    std::string why;
    if (DpComm::unique_id(out, &why)) {
        set_global_error(VB200_ERR_NCCL, why);
        return VB200_ERR_NCCL;
    }
    return VB200_OK;
}

int volta_b200_dp_check(const uint8_t id[128], int32_t world_size, int32_t rank, float *device_buf, int64_t count,
                        void *stream) {
    if (!id || world_size < 1 || rank < 0 || rank >= world_size || count < 0 || (count > 0 && !device_buf)) {
        set_global_error(VB200_ERR_INVALID, "dp_check: bad argument");
        return VB200_ERR_INVALID;
    }
    DpComm comm;
    int rc = comm.init(id, world_size, rank);
    if (!rc && count > 0) rc = comm.all_reduce_sum(device_buf, count, (cudaStream_t)stream);
    if (rc) {
        set_global_error(VB200_ERR_NCCL, comm.error());
        return VB200_ERR_NCCL;
    }
    return VB200_OK;
}

// ---- stand-alone kernel entry points ------------------------------------------------------
int volta_b200_optimizer_apply(int32_t optimizer, float *p, float *s1, float *s2, const float *g, int64_t n,
                               int64_t n_decay, float lr, float weight_decay, float momentum, uint64_t t,
                               void *stream) {
    cudaStream_t s = (cudaStream_t)stream;
    StepScalars sc{};
    sc.lr = lr; sc.beta1 = 0.9f; sc.beta2 = 0.999f; sc.eps = 1e-8f;
    sc.weight_decay = weight_decay; sc.momentum = momentum;
    sc.bc1 = 1.0f - powf(0.9f, (float)t);
    sc.bc2 = 1.0f - powf(0.999f, (float)t);
    StepScalars *d = nullptr;
    if (cudaMalloc(&d, sizeof(StepScalars)) != cudaSuccess) return VB200_ERR_OOM;
    cudaError_t e = launch_set_scalars(d, sc, s);
    if (e == cudaSuccess) e = launch_optimizer(optimizer, p, s1 ? s1 : p, s2 ? s2 : p, g, n, n_decay, d, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(d);
    return e == cudaSuccess ? VB200_OK : VB200_ERR_CUDA;
}

int volta_b200_gemm(int32_t layout, int32_t path, float *C, const float *A, const float *B, int64_t m, int64_t n,
                    int64_t k, void *stream) {
    cudaStream_t s = (cudaStream_t)stream;
    Epilogue e{};
    e.mode = EPI_STORE;
    e.out0 = C;
    e.ld = n;
    cudaError_t err;
    if (path == VB200_GEMM_TENSOR || path == VB200_GEMM_TENSOR_PAIR) {
        if (!gemm_tc_supported(layout, A, B, m, n, k, e)) return VB200_ERR_UNSUPPORTED;
        const bool force_pair = path == VB200_GEMM_TENSOR_PAIR;
        unsigned int *st = nullptr;
        if (cudaMalloc(&st, sizeof(unsigned int)) != cudaSuccess) return VB200_ERR_OOM;
        cudaMemsetAsync(st, 0, sizeof(unsigned int), s);
        float *slabs = nullptr;
        const long long slab_floats = gemm_tc_scratch_floats(layout, m, n, k, force_pair);
        if (slab_floats > 0 && cudaMalloc(&slabs, (size_t)slab_floats * 4) != cudaSuccess) {
            cudaGetLastError();
            slabs = nullptr;   // no room: the unsplit kernel
        }
        err = launch_gemm_tc(layout, A, B, m, n, k, e, st, s, slabs, slabs ? slab_floats : 0, force_pair);
        unsigned int hs = 0;
        if (err == cudaSuccess) err = cudaMemcpyAsync(&hs, st, sizeof hs, cudaMemcpyDeviceToHost, s);
        if (err == cudaSuccess) err = cudaStreamSynchronize(s);
        cudaFree(st);
        if (slabs) cudaFree(slabs);
        if (err == cudaSuccess && hs != 0) return VB200_ERR_DEVICE_WAIT;
    } else if (path == VB200_GEMM_AUTO && layout == GEMM_NN && gemv_rows_supported(B, m, n, k)) {
        err = launch_gemv_rows(A, B, m, n, k, e, s);  // as a handle's forward pass routes at most 8 rows
    } else {
        // same split-K decision as inside a training step, with scratch of this call's own
        float *scratch = nullptr;
        const long long need = ffma_scratch_floats(m, n, k);
        if (need > 0 && cudaMalloc(&scratch, (size_t)need * 4) != cudaSuccess) return VB200_ERR_OOM;
        err = launch_gemm_ffma(layout, A, B, m, n, k, e, s, scratch);
        if (scratch) {
            if (err == cudaSuccess) err = cudaStreamSynchronize(s);
            cudaFree(scratch);
        }
    }
    return err == cudaSuccess ? VB200_OK : VB200_ERR_CUDA;
}

int volta_b200_update_selftest(int32_t optimizer, uint64_t seed, int64_t groups, int32_t wide, uint64_t t, uint64_t counts[3]) {
    if (!counts || groups <= 0 || t == 0 ||
        !(optimizer == VB200_OPT_ADAM || optimizer == VB200_OPT_ADAMW || optimizer == VB200_OPT_ADAGRAD)) {
        set_global_error(VB200_ERR_INVALID, "update_selftest: adam, adamw or adagrad; groups and t positive");
        return VB200_ERR_INVALID;
    }
    StepScalars sc{};
    sc.lr = 1e-3f; sc.beta1 = 0.9f; sc.beta2 = 0.999f; sc.eps = 1e-8f; sc.weight_decay = 0.01f; sc.momentum = 0.9f;
    sc.bc1 = 1.0f - powf(sc.beta1, (float)t);
    sc.bc2 = 1.0f - powf(sc.beta2, (float)t);
    unsigned long long *d = nullptr;
    if (cudaMalloc(&d, 3 * sizeof(unsigned long long)) != cudaSuccess) return VB200_ERR_OOM;
    cudaError_t e = cudaMemset(d, 0, 3 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = launch_update_selftest(optimizer, seed, groups, wide, sc, d, nullptr);
    if (e == cudaSuccess) e = cudaMemcpy(counts, d, 3 * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) {
        set_global_error(VB200_ERR_CUDA, std::string("update_selftest: ") + cudaGetErrorString(e));
        return VB200_ERR_CUDA;
    }
    return VB200_OK;
}

int volta_b200_gemm_route(int32_t layout, int32_t path, int64_t m, int64_t n, int64_t k, int32_t *splits) {
    if (splits) *splits = 1;
    if (m <= 0 || n <= 0 || k <= 0 || layout < GEMM_NN || layout > GEMM_TN) return -VB200_ERR_INVALID;
    // alignment aside (operands of a handle are 1 KiB aligned), the same decisions as run_gemm above
    const long long a_inner = (layout == GEMM_TN) ? m : k, b_inner = (layout == GEMM_NT) ? k : n;
    const bool tc_shape = !((a_inner | b_inner) & 3) && m <= 0x7fffffffLL && n <= 0x7fffffffLL && k <= 0x7fffffffLL;
    if (layout == GEMM_NN && path == VB200_GEMM_AUTO && m <= 8 && gemv_rows_supported(reinterpret_cast<const float *>(uintptr_t(1024)), m, n, k))
        return VB200_ROUTE_SMALL_ROWS;
    if (path != VB200_GEMM_FFMA && tc_shape &&
        (path == VB200_GEMM_TENSOR || path == VB200_GEMM_TENSOR_PAIR || gemm_prefers_tc(m, n, k))) {
        const bool fp = path == VB200_GEMM_TENSOR_PAIR;
        if (splits) *splits = gemm_tc_splits(layout, m, n, k, fp);
        return gemm_tc_uses_pair(layout, m, n, k, fp) ? VB200_ROUTE_TENSOR_PAIR : VB200_ROUTE_TENSOR_SINGLE;
    }
    if (splits) *splits = ffma_splits(m, n, k);
    return VB200_ROUTE_FFMA;
}

int64_t volta_b200_colsum_scratch_floats(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0) return 0;
    return colsum_chunks(rows, cols) * cols;
}

int volta_b200_colsum(float *out, const float *in, int64_t rows, int64_t cols, float *scratch, void *stream) {
    if (!out || !in || !scratch) return VB200_ERR_INVALID;
    cudaError_t e = launch_colsum(out, in, rows, cols, scratch, (cudaStream_t)stream);
    return e == cudaSuccess ? VB200_OK : VB200_ERR_CUDA;
}

}  // extern "C"
