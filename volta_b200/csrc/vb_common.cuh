// Shared declarations of libvolta_b200: error helpers, the epilogue descriptor that every
// GEMM kernel applies to its accumulators, and the device-side activation math.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/volta_b200.h"

#include <stdlib.h>

#include <utility>

namespace vb {

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  The step is a chain of short kernels, each depending on the
// one before; launched this way a kernel's CTAs can be scheduled while its predecessor drains,
// and they block in pdl_wait() until the predecessor has completed and its writes are visible.
// Rule for every kernel launched through launch_pdl: call pdl_wait() before the first access
// to global memory, and pdl_trigger() once the dependent may start being scheduled.
// VOLTA_B200_PDL=0 turns the launch attribute off (the device-side calls are then no-ops).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
    static const bool on = [] { const char *e = getenv("VOLTA_B200_PDL"); return !(e && e[0] == '0'); }();
    return on;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

// ---------------------------------------------------------------------------------------
// Per-device state.  A process may hold handles on several GPUs: function attributes (the
// dynamic shared-memory limit) are set per device, and SM counts differ between devices, so
// neither may be cached per process.
// ---------------------------------------------------------------------------------------
constexpr int kMaxDevices = 64;
inline int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); dev = 0; }
    return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}
// Raises a kernel's dynamic shared-memory limit once per device.
template <typename K>
cudaError_t set_smem_once(K kernel, int bytes, bool (&done)[kMaxDevices]) {
    const int dev = current_device();
    if (done[dev]) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done[dev] = true;
    return e;
}
// Number of SMs of the current device (148 on B200).
inline int device_sm_count() {
    static int sms[kMaxDevices] = {};
    const int dev = current_device();
    if (sms[dev] <= 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) cudaGetLastError();
        sms[dev] = v > 0 ? v : 148;
    }
    return sms[dev];
}

// ---------------------------------------------------------------------------------------
// Activation math, following the reference's generated helpers
// (src/engine/ir/codegen/mlp_train_rust_codegen.rs:563-596, 725-743, 894-916).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ float act_forward(int act, float x) {
    switch (act) {
    case VB200_ACT_RELU: return x > 0.0f ? x : 0.0f;
    case VB200_ACT_SIGMOID: return sigmoidf_(x);
    case VB200_ACT_TANH: return tanhf(x);
    case VB200_ACT_LEAKY_RELU: return x > 0.0f ? x : 0.01f * x;
    case VB200_ACT_SILU: return x * sigmoidf_(x);
    case VB200_ACT_GELU: {
        const float c = 0.7978845608f, k = 0.044715f;
        float v = c * (x + k * x * x * x);
        return 0.5f * x * (1.0f + tanhf(v));
    }
    }
    return x;
}

// `saved` is whatever the forward pass kept for this activation: the pre-activation for
// silu/gelu, the post-activation for relu/leaky (same sign as the pre-activation, so the
// reference's `pre > 0` mask is reproduced exactly) and for sigmoid/tanh (whose
// derivatives the reference also takes from the post-activation).
__device__ __forceinline__ float act_backward(int act, float saved) {
    switch (act) {
    case VB200_ACT_RELU: return saved > 0.0f ? 1.0f : 0.0f;
    case VB200_ACT_SIGMOID: return saved * (1.0f - saved);
    case VB200_ACT_TANH: return 1.0f - saved * saved;
    case VB200_ACT_LEAKY_RELU: return saved > 0.0f ? 1.0f : 0.01f;
    case VB200_ACT_SILU: { float s = sigmoidf_(saved); return s * (1.0f + saved * (1.0f - s)); }
    case VB200_ACT_GELU: {
        const float c = 0.7978845608f, k = 0.044715f;
        float v = c * (saved + k * saved * saved * saved);
        float t = tanhf(v), t2 = 1.0f - t * t;
        return 0.5f * (1.0f + t) + 0.5f * saved * t2 * c * (1.0f + 3.0f * k * saved * saved);
    }
    }
    return 1.0f;
}

// True when backward needs the pre-activation kept separately from the post-activation.
__host__ __device__ inline bool act_needs_pre(int act) { return act == VB200_ACT_SILU || act == VB200_ACT_GELU; }

// ---------------------------------------------------------------------------------------
// Epilogue applied to each accumulator element (row m, column n of the GEMM output).
// ---------------------------------------------------------------------------------------
enum EpiMode {
    EPI_STORE = 0,     // out0[m,n] = acc                                   (dW)
    EPI_BIAS_ACT = 1,  // z = acc + bias[n]; out1[m,n] = z (if out1); out0[m,n] = f(z)   (forward, hidden)
    EPI_BIAS = 2,      // out0[m,n] = acc + bias[n]                         (forward, last layer)
    EPI_DACT = 3,      // out0[m,n] = acc * f'(saved[m,n])                  (dX + activation backward)
    EPI_SGD = 4,       // out0[m,n] = out0[m,n] - lr * acc                  (dW folded into the SGD update,
                       //   the reference's sgd_fused_tn, mlp_train_rust_codegen.rs:321-324, 988)
};

struct Epilogue {
    int mode;
    int act;
    float *out0;        // leading dimension ld
    float *out1;        // optional second output (pre-activation), same ld
    const float *bias;  // [n]
    const float *saved; // [m x n], same ld
    const float *lr;    // EPI_SGD: device pointer to this step's learning rate
    long long ld;

    __device__ __forceinline__ void apply(long long m, long long n, float acc) const {
        long long idx = m * ld + n;
        switch (mode) {
        case EPI_STORE: out0[idx] = acc; break;
        case EPI_BIAS_ACT: {
            float z = acc + bias[n];
            if (out1) out1[idx] = z;
            out0[idx] = act_forward(act, z);
            break;
        }
        case EPI_BIAS: out0[idx] = acc + bias[n]; break;
        case EPI_DACT: out0[idx] = acc * act_backward(act, saved[idx]); break;
        case EPI_SGD: out0[idx] = __fsub_rn(out0[idx], __fmul_rn(*lr, acc)); break;
        }
    }
    // Same for four consecutive columns n..n+3 (idx 16-byte aligned, all in range).
    __device__ __forceinline__ void apply4(long long m, long long n, float4 acc) const {
        long long idx = m * ld + n;
        switch (mode) {
        case EPI_STORE: *reinterpret_cast<float4 *>(out0 + idx) = acc; break;
        case EPI_BIAS_ACT: {
            float4 b = *reinterpret_cast<const float4 *>(bias + n);
            float4 z = make_float4(acc.x + b.x, acc.y + b.y, acc.z + b.z, acc.w + b.w);
            if (out1) *reinterpret_cast<float4 *>(out1 + idx) = z;
            *reinterpret_cast<float4 *>(out0 + idx) =
                make_float4(act_forward(act, z.x), act_forward(act, z.y), act_forward(act, z.z), act_forward(act, z.w));
            break;
        }
        case EPI_BIAS: {
            float4 b = *reinterpret_cast<const float4 *>(bias + n);
            *reinterpret_cast<float4 *>(out0 + idx) = make_float4(acc.x + b.x, acc.y + b.y, acc.z + b.z, acc.w + b.w);
            break;
        }
        case EPI_DACT: {
            float4 s = *reinterpret_cast<const float4 *>(saved + idx);
            *reinterpret_cast<float4 *>(out0 + idx) =
                make_float4(acc.x * act_backward(act, s.x), acc.y * act_backward(act, s.y),
                            acc.z * act_backward(act, s.z), acc.w * act_backward(act, s.w));
            break;
        }
        case EPI_SGD: {
            const float l = *lr;
            float4 w = *reinterpret_cast<const float4 *>(out0 + idx);
            *reinterpret_cast<float4 *>(out0 + idx) =
                make_float4(__fsub_rn(w.x, __fmul_rn(l, acc.x)), __fsub_rn(w.y, __fmul_rn(l, acc.y)),
                            __fsub_rn(w.z, __fmul_rn(l, acc.z)), __fsub_rn(w.w, __fmul_rn(l, acc.w)));
            break;
        }
        }
    }
};

// GEMM operand layouts: C[m x n] = op(A) . op(B)
enum GemmLayout {
    GEMM_NN = 0,  // A[m x k], B[k x n]   forward:  act . W
    GEMM_NT = 1,  // A[m x k], B[n x k]   dX:       delta . W^T
    GEMM_TN = 2,  // A[k x m], B[k x n]   dW:       act^T . delta
};

// Per-step scalars read by the optimizer kernel; written by a one-thread kernel ahead of
// the captured step so that the graph itself never changes.
struct StepScalars {
    float lr;
    float bc1, bc2;       // Adam bias corrections 1 - beta^t (host powf, mlp_train_rust_codegen.rs:811)
    float beta1, beta2;
    float eps;
    float weight_decay;
    float momentum;
    float inv_unused;
    unsigned int epoch;   // step counter, the same on every data-parallel rank (orders the peer barriers)
    unsigned long long rng_base;  // dropout: state of the mask stream before this step's first draw
    unsigned int pad[4];
};
static_assert(sizeof(StepScalars) == 64, "StepScalars is one 64-byte record");

// The dropout mask stream (mlp_train_rust_codegen.rs:773-788): a 64-bit LCG, one draw per element.
constexpr unsigned long long kLcgA = 6364136223846793005ULL, kLcgC = 1442695040888963407ULL;
// State after n more draws.  The map s -> a*s + c composed with itself is s -> a*a*s + (a+1)*c, so the
// draws are applied by the binary digits of n.
__host__ __device__ inline unsigned long long lcg_jump(unsigned long long s, unsigned long long n) {
    unsigned long long a = kLcgA, c = kLcgC;
    while (n) {
        if (n & 1ULL) s = s * a + c;
        c = (a + 1ULL) * c;
        a = a * a;
        n >>= 1;
    }
    return s;
}

// ---------------------------------------------------------------------------------------
// Kernel launchers (defined in the .cu files of this directory).
// ---------------------------------------------------------------------------------------
// `scratch` (ffma_scratch_floats(m, n, k) floats, may be null) enables deterministic split-K for
// shapes whose output gives too few tiles to occupy the GPU.
cudaError_t launch_gemm_ffma(int layout, const float *A, const float *B, long long m, long long n, long long k,
                             const Epilogue &epi, cudaStream_t s, float *scratch = nullptr);
int ffma_splits(long long m, long long n, long long k);
long long ffma_scratch_floats(long long m, long long n, long long k);
// Shape heuristic: true when the tensor-core kernel is expected to beat the FFMA path.
bool gemm_prefers_tc(long long m, long long n, long long k);
// Returns cudaErrorNotSupported when the shape/alignment cannot take the tensor path.
// `scratch` (gemm_tc_scratch_floats floats, may be null) lets a GEMM whose tiles fill the last wave badly
// split K over concurrent CTAs; the slabs are then added in split order by launch_splitk_reduce.
// `force_pair` restricts the choice to the CTA-pair kernel (outputs of at least 256 x 256).  Kernel and
// split count are functions of (m, n, k, force_pair) alone.
cudaError_t launch_gemm_tc(int layout, const float *A, const float *B, long long m, long long n, long long k,
                           const Epilogue &epi, unsigned int *status_word, cudaStream_t s, float *scratch = nullptr,
                           long long scratch_floats = 0, bool force_pair = false);
int gemm_tc_splits(int layout, long long m, long long n, long long k, bool force_pair = false);
bool gemm_tc_uses_pair(int layout, long long m, long long n, long long k, bool force_pair = false);
long long gemm_tc_scratch_floats(int layout, long long m, long long n, long long k, bool force_pair = false);
// out = epilogue(sum over z of partial[z][m x n]), z ascending
cudaError_t launch_splitk_reduce(const float *partial, long long m, long long n, int splits, const Epilogue &epi,
                                 cudaStream_t s);
cudaError_t launch_gemm_tc2(int layout, const float *A, const float *B, long long m, long long n, long long k,
                            const Epilogue &epi, unsigned int *status_word, cudaStream_t s, int splits = 1);
cudaError_t launch_gemm_tc3(int layout, const float *A, const float *B, long long m, long long n, long long k,
                            const Epilogue &epi, unsigned int *status_word, cudaStream_t s, int splits = 1);
bool gemm_tc_supported(int layout, const float *A, const float *B, long long m, long long n, long long k,
                       const Epilogue &epi);

// Forward GEMM (NN) for at most 8 rows: one pass over W by clusters of CTAs that reduce through
// distributed shared memory (vb_gemv.cu).  x may live in pinned host memory.
bool gemv_rows_supported(const float *W, long long m, long long n, long long k);
cudaError_t launch_gemv_rows(const float *x, const float *W, long long m, long long n, long long k, const Epilogue &epi,
                             cudaStream_t s);

cudaError_t launch_optimizer(int optimizer, float *p, float *s1, float *s2, const float *g, long long n,
                             long long n_decay, const StepScalars *sc, cudaStream_t s);
cudaError_t launch_set_scalars(StepScalars *dst, StepScalars v, cudaStream_t s);
// update_rows (the persistent step kernel's optimizer) against update_one on `groups` seeded groups of four
// elements; counts[0..2] (device, zeroed by the caller) += differing elements, core groups, library groups.
cudaError_t launch_update_selftest(int optimizer, unsigned long long seed, long long groups, int wide, const StepScalars &sc,
                                   unsigned long long *counts, cudaStream_t s);
// first_bad[0..3] = min(first_bad[r], smallest index of an inf/NaN in g[0..n_grads), p, s1, s2 [0..n));
// null regions are skipped; the caller presets the four words to all ones.
cudaError_t launch_finite_guard(const float *p, const float *g, const float *s1, const float *s2, long long n,
                                long long n_grads, unsigned long long *first_bad, cudaStream_t s);

// ---- fused data-parallel update over peer memory (vb_dp_fused.cu)
constexpr int kMaxPeers = 8;
struct PeerTable {
    char *base[kMaxPeers];   // every rank's arena, mapped into this process (own arena at [rank])
};
// One barrier among the ranks: write `*epoch * stride + index` into slot `rank` of every peer's flag
// array, then wait until all of this rank's slots have reached it - for at most wait_ns, after which
// the DP-barrier bit is set in *status.  Once that bit is set (by this or an earlier launch) the
// kernel returns at once without touching a peer: the missing rank's memory may be gone.
cudaError_t launch_dp_barrier(const PeerTable &peers, long long flags_off, int world, int rank,
                              const StepScalars *scalars, unsigned stride, unsigned index, unsigned int *status,
                              unsigned long long wait_ns, cudaStream_t s);
// For the floats [seg_begin, seg_begin + seg_len) of the flat layout: this rank sums its 1/world share
// of every rank's gradients in rank order, applies the optimizer to its share of the parameters, and
// writes the new parameters into every rank's arena.  Does nothing once the DP-barrier bit of *status
// is set: after a barrier gave up, some rank's gradients are missing or stale and its arena may be gone.
cudaError_t launch_dp_reduce_update(int optimizer, const PeerTable &peers, long long params_off, long long grads_off,
                                    long long s1_off, long long s2_off, long long seg_begin, long long seg_len,
                                    long long n_decay, int world, int rank, const StepScalars *scalars,
                                    long long loss_off, const unsigned int *status, cudaStream_t s);
// Exchange by copy: for the floats [seg_begin, seg_begin + seg_len) this rank adds the `world` gradient copies
// (its own `grads`, and for every other rank q the receive slot recv + q * slot_floats that rank q's copy
// engines filled) in rank order, stores the sum back into `grads` and applies the optimizer to the whole
// segment.  With loss_index >= 0 the loss sums at that index of every copy are added likewise into
// grads[loss_index + 1].  Local memory only.  Does nothing once the DP-barrier bit of *status is set.
cudaError_t launch_dp_gather_update(int optimizer, float *params, float *s1, float *s2, float *grads, const float *recv,
                                    long long slot_floats, long long seg_begin, long long seg_len, long long n_decay,
                                    int world, int rank, const StepScalars *scalars, long long loss_index,
                                    const unsigned int *status, cudaStream_t s);
constexpr unsigned kStatusDpBarrier = 64u;   // status-word bit: a data-parallel barrier wait ran out

// ---- the whole step as one persistent kernel, batches of at most 64 rows (vb_step_small.cu)
constexpr int kSmallStepMaxLayers = 16;
struct SmallStepLayer {
    int r, c;                  // W is [r x c]
    long long off_w, off_b;    // floats from the start of the flat parameter / gradient / state regions
    const float *act_in;       // [B x r]
    float *act_out;            // [B x c]
    float *pre_out;            // [B x c] or null: the pre-activation, where backward needs it
    float *delta;              // [B x c]
    const float *saved_prev;   // [B x r]: what the previous layer's activation derivative takes; null for layer 0
    float *delta_prev;         // [B x r]; null for layer 0
};
struct SmallStepArgs {
    int n, B, act, opt;
    int forward_only;          // 1: stop after the last layer's outputs (inference); B is then the row count
    float *params, *grads, *s1, *s2;
    long long n_params_padded;
    const float *y;            // [B x L_n]
    float *loss_sum, *loss_partials;   // one float; one float per CTA
    float nt_global;
    StepScalars scalars;       // this step's learning rate and optimizer constants, by value
    unsigned int *barrier;     // {arrival word, -, abort}
    unsigned int *status;
    float *host_loss;          // pinned host memory the kernel stores the loss sum and the status word to
    unsigned int *host_status; //   at its end (either may be null)
    SmallStepLayer L[kSmallStepMaxLayers];
};
bool small_step_shape_ok(const int *layers, int n_sizes, int batch, int clusters);
int small_step_grid(int optimizer, int *cluster);
cudaError_t launch_small_step(const SmallStepArgs &args, int grid, int cluster, cudaStream_t s);

long long colsum_chunks(long long rows, long long cols);
// out[j] = sum_rows in[row, j] * (row_weight ? row_weight[row] : 1), fixed order
cudaError_t launch_colsum(float *out, const float *in, long long rows, long long cols, float *scratch, cudaStream_t s,
                          const float *row_weight = nullptr);
// out[row] = in[row, :] . w + bias[0]
cudaError_t launch_rowdot(float *out, const float *in, const float *w, const float *bias, long long rows,
                          long long cols, cudaStream_t s);

// ---- row-wise kernels of the optional stages (vb_options.cu)
struct RowFwd {
    int softmax;                 // 1: x holds bias-added pre-activations and leaves as their row softmax
    const float *ln_g, *ln_b;    // LayerNorm scale/shift [cols], or null
    float *ln_is;                // [rows] 1/sqrt(var + eps) kept for backward
    float dropout_p;             // 0 = no dropout
    unsigned char *mask;         // [rows x cols] keep flags kept for backward
    unsigned long long draw_off; // draws of this step that precede row 0 of this call
};
struct RowBwd {
    int act;                     // VB200_ACT_*
    const float *a1;             // the layer's stored output (after every stage) [rows x cols]
    const float *saved;          // what act_backward takes (pre-activation or a1); unused for softmax
    const float *ln_g, *ln_b, *ln_is;  // or null
    float dropout_p;
    const unsigned char *mask;
};
// Largest hidden width the row kernels take (one row is staged in shared memory).
constexpr int kRowMaxCols = 51200;
cudaError_t launch_row_forward(float *x, long long rows, int cols, const RowFwd &o, const StepScalars *sc, cudaStream_t s);
cudaError_t launch_row_backward(float *delta, long long rows, int cols, const RowBwd &o, cudaStream_t s);
// out[0..cols) = sum_rows dout*xhat, out[cols..2cols) = sum_rows dout, xhat rebuilt from a1 as the
// reference does; scratch holds colsum_chunks(rows, cols) * 2 * cols floats
cudaError_t launch_ln_param_grads(float *out, const float *dout, const float *a1, const float *g, const float *b,
                                  long long rows, int cols, float *scratch, cudaStream_t s);
// partial[0..loss_blocks(n)) = fixed-order block sums of v*v
cudaError_t launch_sumsq_partials(float *partial, const float *v, long long n, cudaStream_t s);
// *out = sum of partial[0..nblocks) in a fixed order
cudaError_t launch_sum_partials(float *out, const float *partial, long long nblocks, cudaStream_t s);
// v *= clip/sqrt(*norm_sq) when sqrt(*norm_sq) > clip, else untouched
cudaError_t launch_clip_scale(float *v, long long n, const float *norm_sq, float clip, cudaStream_t s);

// out[row, k] = delta[row] * w[k] * f'(saved[row, k])  (saved may be null: no derivative factor)
cudaError_t launch_rank1_dx(float *out, const float *delta, const float *w, const float *saved, int act, long long rows,
                            long long cols, cudaStream_t s);

long long loss_blocks(long long nt);
// delta[k] = 2*(out[k]-y[k])/nt_global ; *loss_sum = sum_k (out[k]-y[k])^2 (fixed order)
cudaError_t launch_mse_seed(float *delta, float *loss_sum, const float *out, const float *y, long long nt,
                            float nt_global, float *scratch, cudaStream_t s);

}  // namespace vb
