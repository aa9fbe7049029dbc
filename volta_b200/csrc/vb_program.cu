// Runtime-backend slice: a scheduled graph of tensor ops compiled onto one device arena and one
// CUDA graph.  It is what a `B200Backend` for Volta's runtime (`trait Backend`,
// src/engine/ir/backend.rs:24-69) would sit on: compile(plan) -> volta_b200_program_compile,
// execute_value / execute_terminal -> bind + run + fetch, apply_gradients -> volta_b200_program_update.
// The op set is the one the runtime's MLP training graphs use (src/engine/ir/lowering.rs:90-140 forward,
// src/engine/ir/autograd.rs:119-450 backward): Input, Parameter, ConstTensor, Add, Sub, Mul, Div, Neg,
// Transpose, MatMul, Relu, ReluBackward, Sigmoid, SigmoidBackward, Gelu, GeluBackward, Softmax, Log, Exp,
// ReduceSum, ReduceMean, SoftmaxCrossEntropyLossFromLogits, Reshape, Identity, Output - semantics as src/engine/ir/interpreter.rs:680-880 and
// src/engine/ir/kernels/{activations,reduce,utils}.rs (numpy-style broadcasting of rank <= 2).
//
// Where the reference interprets node by node with a host tensor per value (and its CUDA executor moves
// every operand over PCIe per op, src/engine/ir/cuda/executor.rs), here
//   * parameters and inputs stay resident; temporaries are placed by liveness in one arena
//     (the planner of vb_arena.h, i.e. the scheme of src/engine/ir/memory_planner.rs:47-144);
//   * Transpose feeding MatMul becomes the GEMM's operand layout (nothing is moved);
//   * MatMul -> Add(row bias) -> Relu/Sigmoid/Gelu becomes one GEMM with a fused epilogue, and
//     ReluBackward/GeluBackward of a MatMul result becomes the epilogue of that GEMM;
//   * the whole schedule is captured once into a CUDA graph and replayed per run.
#include <math.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "vb_arena.h"
#include "vb_common.cuh"
#include "vb_optimizer.cuh"

using namespace vb;

namespace {

// ---------------------------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------------------------
enum { BIN_ADD = 0, BIN_SUB, BIN_MUL, BIN_DIV, BIN_RELU_BWD, BIN_SIGMOID_BWD, BIN_GELU_BWD };
enum { UN_NEG = 0, UN_RELU, UN_SIGMOID, UN_GELU, UN_LOG, UN_EXP };

__device__ __forceinline__ float bin_apply(int op, float a, float b) {
    switch (op) {
    case BIN_ADD: return a + b;
    case BIN_SUB: return a - b;
    case BIN_MUL: return a * b;
    case BIN_DIV: return a / b;
    // the backward ops take the activation's INPUT and the upstream gradient (kernels/activations.rs:34-118, 168-200)
    case BIN_RELU_BWD: return a > 0.0f ? b : 0.0f;
    case BIN_SIGMOID_BWD: { float s = sigmoidf_(a); return b * s * (1.0f - s); }
    case BIN_GELU_BWD: return b * act_backward(VB200_ACT_GELU, a);
    }
    return 0.0f;
}

__device__ __forceinline__ float un_apply(int op, float a) {
    switch (op) {
    case UN_NEG: return -a;
    case UN_RELU: return a > 0.0f ? a : 0.0f;
    case UN_SIGMOID: return sigmoidf_(a);
    case UN_GELU: return act_forward(VB200_ACT_GELU, a);
    case UN_LOG: return logf(a);
    case UN_EXP: return expf(a);
    }
    return a;
}

// out[i, j] = f(a[i*ar + j*ac], b[i*br + j*bc]) over an R x C output; a stride of 0 broadcasts
__global__ void __launch_bounds__(256) binary_kernel(int op, float *__restrict__ out, const float *__restrict__ a,
                                                     const float *__restrict__ b, long long R, long long C, long long ar,
                                                     long long ac, long long br, long long bc) {
    pdl_wait();
    pdl_trigger();
    const long long n = R * C, stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
        const long long i = e / C, j = e - i * C;
        out[e] = bin_apply(op, a[i * ar + j * ac], b[i * br + j * bc]);
    }
}

__global__ void __launch_bounds__(256) unary_kernel(int op, float *__restrict__ out, const float *__restrict__ a, long long n) {
    pdl_wait();
    pdl_trigger();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) out[e] = un_apply(op, a[e]);
}

// out[C x R] = in[R x C]^T through a padded 32 x 32 tile
__global__ void __launch_bounds__(256) transpose_kernel(float *__restrict__ out, const float *__restrict__ in, long long R,
                                                        long long C) {
    __shared__ float tile[32][33];
    pdl_wait();
    pdl_trigger();
    const long long c0 = (long long)blockIdx.x * 32, r0 = (long long)blockIdx.y * 32;
    for (int y = threadIdx.y; y < 32; y += 8) {
        const long long r = r0 + y, c = c0 + threadIdx.x;
        if (r < R && c < C) tile[y][threadIdx.x] = in[r * C + c];
    }
    __syncthreads();
    for (int y = threadIdx.y; y < 32; y += 8) {
        const long long c = c0 + y, r = r0 + threadIdx.x;
        if (r < R && c < C) out[c * R + r] = tile[threadIdx.x][y];
    }
}

// out[row] = scale * sum_j in[row, j]; one warp per row, fixed lane shares and shuffle tree
__global__ void __launch_bounds__(256) rowsum_kernel(float *__restrict__ out, const float *__restrict__ in, long long R,
                                                     long long C, float scale) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long row = (((long long)blockIdx.x * blockDim.x) + threadIdx.x) >> 5; row < R; row += warps) {
        float acc = 0.0f;
        for (long long c = lane; c < C; c += 32) acc += in[row * C + c];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
        if (lane == 0) out[row] = acc * scale;
    }
}

// block partials of a plain sum (4096 elements per block), then one block adds them in order
__global__ void __launch_bounds__(256) sum_blocks_kernel(float *__restrict__ partial, const float *__restrict__ v, long long n) {
    __shared__ float sm[8];
    pdl_wait();
    pdl_trigger();
    const long long base = (long long)blockIdx.x * 4096;
    float acc = 0.0f;
#pragma unroll 4
    for (int j = 0; j < 16; ++j) {
        const long long k = base + j * 256 + threadIdx.x;
        if (k < n) acc += v[k];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = sm[0];
        for (int j = 1; j < 8; ++j) t += sm[j];
        partial[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(256) sum_final_kernel(float *__restrict__ out, const float *__restrict__ partial,
                                                        long long nblocks, float scale) {
    __shared__ float sm[8];
    pdl_wait();
    pdl_trigger();
    float acc = 0.0f;
    for (long long k = threadIdx.x; k < nblocks; k += 256) acc += partial[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = sm[0];
        for (int j = 1; j < 8; ++j) t += sm[j];
        *out = t * scale;
    }
}

__global__ void __launch_bounds__(256) scale_kernel(float *__restrict__ v, long long n, float scale) {
    pdl_wait();
    pdl_trigger();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) v[e] *= scale;
}

// Per-row softmax cross-entropy from logits (interpreter.rs:776-815): loss[row] = -sum_j t[j] * (x[j] - lse(x)),
// lse = max + ln(sum exp(x - max)).  One warp per row; the mean over rows follows as a fixed-order sum.
__global__ void __launch_bounds__(256) xent_rows_kernel(float *__restrict__ row_loss, const float *__restrict__ logits,
                                                        const float *__restrict__ targets, long long R, long long C) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long row = (((long long)blockIdx.x * blockDim.x) + threadIdx.x) >> 5; row < R; row += warps) {
        const float *x = logits + row * C, *t = targets + row * C;
        float mx = -INFINITY;
        for (long long c = lane; c < C; c += 32) mx = fmaxf(mx, x[c]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float se = 0.0f;
        for (long long c = lane; c < C; c += 32) se += expf(x[c] - mx);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
        const float lse = mx + logf(se);
        float acc = 0.0f;
        for (long long c = lane; c < C; c += 32) acc -= t[c] * (x[c] - lse);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
        if (lane == 0) row_loss[row] = acc;
    }
}

int grid_for(long long n) {
    long long want = (n + 255) / 256;
    return (int)std::max<long long>(1, std::min<long long>(want, 148 * 8));
}

// ---------------------------------------------------------------------------------------------
// program
// ---------------------------------------------------------------------------------------------
struct PValue {
    int id = -1, kind = -1;
    std::vector<int> in;           // indices into values
    std::vector<int64_t> shape;
    std::vector<float> attrs;
    std::vector<float> const_data;
    long long R = 1, C = 1, count = 1;
    int alias = -1;                // shares the storage of this value
    int buf = -1;                  // plan buffer of a storage-owning value
    bool keep = false;             // marked as an output: stays valid after a run
    bool produced = false;         // some launch (or a binding) writes it
    float *dev = nullptr;
};

enum LaunchKind { L_BINARY, L_UNARY, L_TRANSPOSE, L_GEMM, L_SOFTMAX, L_REDUCE, L_XENT };

struct Launch {
    LaunchKind kind;
    int op = 0;
    int out = -1, a = -1, b = -1;
    int layout = GEMM_NN, epi_mode = EPI_STORE, epi_act = 0, bias = -1, out1 = -1, saved = -1;
    int axis = -1;
    float scale = 1.0f;
    long long m = 0, n = 0, k = 0;
};

bool is_source(int kind) { return kind == VB200_OP_INPUT || kind == VB200_OP_PARAMETER || kind == VB200_OP_CONST; }

}  // namespace

struct vb200_program {
    std::vector<PValue> values;
    std::map<int, int> index_of;   // ValueId -> position in values
    std::vector<Launch> launches;
    ArenaPlan plan;
    char *arena = nullptr;
    int64_t arena_bytes = 0;
    float *reduce_scratch = nullptr, *gemm_scratch = nullptr;
    long long gemm_scratch_floats = 0;
    unsigned int *status_word = nullptr;
    StepScalars *scalars = nullptr;
    cudaStream_t stream = nullptr;
    cudaGraphExec_t graph = nullptr;
    bool compiled = false, attempted = false, fuse = true;
    std::map<int, std::pair<float *, float *>> opt_state;   // parameter index -> moments (outside the arena)
    std::string error;

    int fail(int code, const std::string &msg) {
        error = msg;
        return code;
    }
    int root(int v) const {
        while (values[(size_t)v].alias >= 0) v = values[(size_t)v].alias;
        return v;
    }
};

namespace {

#define VP_CUDA(p, expr)                                                                                       \
    do {                                                                                                       \
        cudaError_t _e = (expr);                                                                               \
        if (_e != cudaSuccess)                                                                                 \
            return (p)->fail(_e == cudaErrorMemoryAllocation ? VB200_ERR_OOM : VB200_ERR_CUDA,                 \
                             std::string(#expr) + ": " + cudaGetErrorString(_e));                              \
    } while (0)

bool to_2d(const std::vector<int64_t> &shape, long long *R, long long *C) {
    if (shape.size() > 2) return false;
    *R = shape.size() == 2 ? shape[0] : 1;
    *C = shape.empty() ? 1 : shape.back();
    return *R >= 0 && *C >= 0;
}

// strides of an operand of 2-D extent (r, c) read under an R x C output; false when it does not broadcast
bool bcast(long long r, long long c, long long R, long long C, long long *sr, long long *sc) {
    if ((r != R && r != 1) || (c != C && c != 1)) return false;
    *sr = r == 1 ? 0 : c;
    *sc = c == 1 ? 0 : 1;
    return true;
}

int act_of(int kind) {
    switch (kind) {
    case VB200_OP_RELU: return VB200_ACT_RELU;
    case VB200_OP_SIGMOID: return VB200_ACT_SIGMOID;
    case VB200_OP_GELU: return VB200_ACT_GELU;
    }
    return -1;
}

std::string describe(const PValue &v) {
    std::string s = "value " + std::to_string(v.id) + " (op " + std::to_string(v.kind) + ", shape [";
    for (size_t i = 0; i < v.shape.size(); ++i) s += (i ? "," : "") + std::to_string(v.shape[i]);
    return s + "])";
}

// Shape rules of the ops, as the reference's shape inference has them (src/engine/ir/shape_inference.rs)
int check_node(vb200_program *p, const PValue &v) {
    auto in = [&](int k) -> const PValue & { return p->values[(size_t)v.in[(size_t)k]]; };
    auto need = [&](size_t n) { return v.in.size() == n; };
    switch (v.kind) {
    case VB200_OP_INPUT:
    case VB200_OP_PARAMETER:
    case VB200_OP_CONST:
        if (!need(0)) return p->fail(VB200_ERR_INVALID, describe(v) + " takes no inputs");
        return VB200_OK;
    case VB200_OP_ADD: case VB200_OP_SUB: case VB200_OP_MUL: case VB200_OP_DIV: {
        if (!need(2)) return p->fail(VB200_ERR_INVALID, describe(v) + " takes two inputs");
        long long s;
        if (!bcast(in(0).R, in(0).C, v.R, v.C, &s, &s) || !bcast(in(1).R, in(1).C, v.R, v.C, &s, &s) ||
            v.R != std::max(in(0).R, in(1).R) || v.C != std::max(in(0).C, in(1).C))
            return p->fail(VB200_ERR_INVALID, "Cannot broadcast the operands of " + describe(v));
        return VB200_OK;
    }
    case VB200_OP_RELU_BACKWARD: case VB200_OP_SIGMOID_BACKWARD: case VB200_OP_GELU_BACKWARD:
        if (!need(2) || in(0).shape != v.shape || in(1).shape != v.shape)
            return p->fail(VB200_ERR_INVALID, "Shape mismatch in " + describe(v));
        return VB200_OK;
    case VB200_OP_NEG: case VB200_OP_RELU: case VB200_OP_SIGMOID: case VB200_OP_GELU: case VB200_OP_LOG: case VB200_OP_EXP:
    case VB200_OP_IDENTITY: case VB200_OP_OUTPUT:
        if (!need(1) || in(0).shape != v.shape) return p->fail(VB200_ERR_INVALID, "Shape mismatch in " + describe(v));
        return VB200_OK;
    case VB200_OP_SOFTMAX_XENT:
        if (!need(2) || in(0).shape.size() != 2 || in(0).shape != in(1).shape || !v.shape.empty())
            return p->fail(VB200_ERR_INVALID, "Shape mismatch in SoftmaxCrossEntropyLossFromLogits: " + describe(v));
        return VB200_OK;
    case VB200_OP_RESHAPE:
        if (!need(1) || in(0).count != v.count) return p->fail(VB200_ERR_INVALID, "Reshape changes the element count: " + describe(v));
        return VB200_OK;
    case VB200_OP_SOFTMAX:
        if (!need(1) || in(0).shape != v.shape || v.shape.empty())
            return p->fail(VB200_ERR_INVALID, "Softmax expects 1D or 2D: " + describe(v));
        if (v.C > kRowMaxCols) return p->fail(VB200_ERR_UNSUPPORTED, "Softmax rows longer than 51200: " + describe(v));
        return VB200_OK;
    case VB200_OP_TRANSPOSE:
        if (!need(1) || in(0).shape.size() != 2 || v.shape.size() != 2 || v.R != in(0).C || v.C != in(0).R)
            return p->fail(VB200_ERR_INVALID, "Transpose expects a 2D operand: " + describe(v));
        return VB200_OK;
    case VB200_OP_MATMUL:
        if (!need(2) || in(0).shape.size() != 2 || in(1).shape.size() != 2 || v.shape.size() != 2 || in(0).C != in(1).R ||
            v.R != in(0).R || v.C != in(1).C)
            return p->fail(VB200_ERR_INVALID, "MatMul shape mismatch: " + describe(v));
        return VB200_OK;
    case VB200_OP_REDUCE_SUM: case VB200_OP_REDUCE_MEAN: {
        if (!need(1) || v.attrs.size() < 2) return p->fail(VB200_ERR_INVALID, describe(v) + " needs one input and the attributes axis, keepdims");
        const int axis = (int)v.attrs[0];
        const bool keep = v.attrs[1] != 0.0f;
        const std::vector<int64_t> &s = in(0).shape;
        std::vector<int64_t> want;
        if (axis < 0) {
            if (keep) want.assign(s.size(), 1);
        } else {
            if ((size_t)axis >= s.size()) return p->fail(VB200_ERR_INVALID, "reduce axis out of range: " + describe(v));
            for (size_t d = 0; d < s.size(); ++d)
                if ((int)d != axis) want.push_back(s[d]);
                else if (keep) want.push_back(1);
        }
        if (want != v.shape) return p->fail(VB200_ERR_INVALID, "reduce output shape mismatch: " + describe(v));
        return VB200_OK;
    }
    }
    return p->fail(VB200_ERR_UNSUPPORTED, "unsupported op kind in " + describe(v));
}

cudaError_t gemm(vb200_program *p, int layout, const float *A, const float *B, long long m, long long n, long long k,
                 const Epilogue &e) {
    if (layout == GEMM_NN && gemv_rows_supported(B, m, n, k)) return launch_gemv_rows(A, B, m, n, k, e, p->stream);
    if (gemm_tc_supported(layout, A, B, m, n, k, e) && gemm_prefers_tc(m, n, k))
        return launch_gemm_tc(layout, A, B, m, n, k, e, p->status_word, p->stream, p->gemm_scratch, p->gemm_scratch_floats);
    return launch_gemm_ffma(layout, A, B, m, n, k, e, p->stream, p->gemm_scratch);
}

int enqueue(vb200_program *p) {
    cudaStream_t s = p->stream;
    auto dev = [&](int v) -> float * { return v < 0 ? nullptr : p->values[(size_t)p->root(v)].dev; };
    for (const Launch &l : p->launches) {
        const PValue &o = p->values[(size_t)l.out];
        switch (l.kind) {
        case L_BINARY: {
            const PValue &a = p->values[(size_t)l.a], &b = p->values[(size_t)l.b];
            long long ar = 0, ac = 0, br = 0, bc = 0;
            bcast(a.R, a.C, o.R, o.C, &ar, &ac);
            bcast(b.R, b.C, o.R, o.C, &br, &bc);
            VP_CUDA(p, launch_pdl(binary_kernel, dim3(grid_for(o.count)), dim3(256), 0, s, l.op, dev(l.out),
                                  (const float *)dev(l.a), (const float *)dev(l.b), o.R, o.C, ar, ac, br, bc));
            break;
        }
        case L_UNARY:
            VP_CUDA(p, launch_pdl(unary_kernel, dim3(grid_for(o.count)), dim3(256), 0, s, l.op, dev(l.out),
                                  (const float *)dev(l.a), o.count));
            break;
        case L_TRANSPOSE: {
            const PValue &a = p->values[(size_t)l.a];
            dim3 grid((unsigned)((a.C + 31) / 32), (unsigned)((a.R + 31) / 32));
            VP_CUDA(p, launch_pdl(transpose_kernel, grid, dim3(32, 8), 0, s, dev(l.out), (const float *)dev(l.a), a.R, a.C));
            break;
        }
        case L_GEMM: {
            Epilogue e{};
            e.mode = l.epi_mode;
            e.act = l.epi_act;
            e.out0 = dev(l.out);
            e.out1 = dev(l.out1);
            e.bias = dev(l.bias);
            e.saved = dev(l.saved);
            e.ld = l.n;
            VP_CUDA(p, gemm(p, l.layout, dev(l.a), dev(l.b), l.m, l.n, l.k, e));
            break;
        }
        case L_SOFTMAX: {
            VP_CUDA(p, cudaMemcpyAsync(dev(l.out), dev(l.a), (size_t)o.count * 4, cudaMemcpyDeviceToDevice, s));
            RowFwd rf{};
            rf.softmax = 1;
            VP_CUDA(p, launch_row_forward(dev(l.out), o.R, (int)o.C, rf, p->scalars, s));
            break;
        }
        case L_XENT: {
            const PValue &a = p->values[(size_t)l.a];
            float *rows = p->reduce_scratch, *blocks = p->reduce_scratch + a.R;
            const long long want = (a.R + 7) / 8, nb = loss_blocks(a.R);
            VP_CUDA(p, launch_pdl(xent_rows_kernel, dim3((unsigned)std::max<long long>(1, std::min<long long>(want, 148 * 8))), dim3(256),
                                  0, s, rows, (const float *)dev(l.a), (const float *)dev(l.b), a.R, a.C));
            VP_CUDA(p, launch_pdl(sum_blocks_kernel, dim3((unsigned)nb), dim3(256), 0, s, blocks, (const float *)rows, a.R));
            VP_CUDA(p, launch_pdl(sum_final_kernel, dim3(1), dim3(256), 0, s, dev(l.out), (const float *)blocks, nb,
                                  1.0f / (float)a.R));   // mean over the batch
            break;
        }
        case L_REDUCE: {
            const PValue &a = p->values[(size_t)l.a];
            if (l.axis < 0) {  // everything -> one number
                const long long nb = loss_blocks(a.count);
                VP_CUDA(p, launch_pdl(sum_blocks_kernel, dim3((unsigned)nb), dim3(256), 0, s, p->reduce_scratch,
                                      (const float *)dev(l.a), a.count));
                VP_CUDA(p, launch_pdl(sum_final_kernel, dim3(1), dim3(256), 0, s, dev(l.out), (const float *)p->reduce_scratch, nb,
                                      l.scale));
            } else if (l.axis == 0) {  // over rows: the bias-gradient reduction
                VP_CUDA(p, launch_colsum(dev(l.out), dev(l.a), a.R, a.C, p->reduce_scratch, s));
                if (l.scale != 1.0f)
                    VP_CUDA(p, launch_pdl(scale_kernel, dim3(grid_for(a.C)), dim3(256), 0, s, dev(l.out), a.C, l.scale));
            } else {  // over columns
                const long long want = (a.R + 7) / 8;
                VP_CUDA(p, launch_pdl(rowsum_kernel, dim3((unsigned)std::max<long long>(1, std::min<long long>(want, 148 * 8))),
                                      dim3(256), 0, s, dev(l.out), (const float *)dev(l.a), a.R, a.C, l.scale));
            }
            break;
        }
        }
    }
    return VB200_OK;
}

void release(vb200_program *p) {
    if (p->graph) cudaGraphExecDestroy(p->graph);
    p->graph = nullptr;
    if (p->arena) cudaFree(p->arena);
    p->arena = nullptr;
    for (auto &kv : p->opt_state) {
        if (kv.second.first) cudaFree(kv.second.first);
        if (kv.second.second) cudaFree(kv.second.second);
    }
    p->opt_state.clear();
    if (p->stream) cudaStreamDestroy(p->stream);
    p->stream = nullptr;
}

// Builds the launch list from the scheduled nodes, folding what can be folded.
int lower(vb200_program *p) {
    const int nv = (int)p->values.size();
    std::vector<std::vector<int>> users((size_t)nv);
    for (int v = 0; v < nv; ++v)
        for (int in : p->values[(size_t)v].in) users[(size_t)in].push_back(v);
    std::vector<char> done((size_t)nv, 0);   // produced by an earlier fused launch
    // a Transpose is materialised unless every user is a MatMul that takes it as an operand layout
    auto folds_into = [&](int t, int mm) {
        const PValue &m = p->values[(size_t)mm];
        if (!p->fuse || m.kind != VB200_OP_MATMUL) return false;
        const bool at = m.in[0] == t, bt = m.in[1] == t;
        if (at && bt) return false;
        // with both operands transposed only the right one is folded
        if (at && p->values[(size_t)m.in[1]].kind == VB200_OP_TRANSPOSE) return false;
        return true;
    };
    p->launches.clear();
    for (int v = 0; v < nv; ++v) {
        PValue &val = p->values[(size_t)v];
        if (done[(size_t)v] || is_source(val.kind)) continue;
        Launch l{};
        l.out = v;
        switch (val.kind) {
        case VB200_OP_IDENTITY:
        case VB200_OP_OUTPUT:
        case VB200_OP_RESHAPE:
            val.alias = val.in[0];
            continue;
        case VB200_OP_ADD: case VB200_OP_SUB: case VB200_OP_MUL: case VB200_OP_DIV:
        case VB200_OP_RELU_BACKWARD: case VB200_OP_SIGMOID_BACKWARD: case VB200_OP_GELU_BACKWARD:
            l.kind = L_BINARY;
            l.op = val.kind == VB200_OP_ADD ? BIN_ADD : val.kind == VB200_OP_SUB ? BIN_SUB : val.kind == VB200_OP_MUL ? BIN_MUL
                   : val.kind == VB200_OP_DIV ? BIN_DIV : val.kind == VB200_OP_RELU_BACKWARD ? BIN_RELU_BWD
                   : val.kind == VB200_OP_SIGMOID_BACKWARD ? BIN_SIGMOID_BWD : BIN_GELU_BWD;
            l.a = val.in[0];
            l.b = val.in[1];
            break;
        case VB200_OP_NEG: case VB200_OP_RELU: case VB200_OP_SIGMOID: case VB200_OP_GELU: case VB200_OP_LOG: case VB200_OP_EXP:
            l.kind = L_UNARY;
            l.op = val.kind == VB200_OP_NEG ? UN_NEG : val.kind == VB200_OP_RELU ? UN_RELU : val.kind == VB200_OP_SIGMOID ? UN_SIGMOID
                   : val.kind == VB200_OP_GELU ? UN_GELU : val.kind == VB200_OP_LOG ? UN_LOG : UN_EXP;
            l.a = val.in[0];
            break;
        case VB200_OP_SOFTMAX:
            l.kind = L_SOFTMAX;
            l.a = val.in[0];
            break;
        case VB200_OP_SOFTMAX_XENT:
            l.kind = L_XENT;
            l.a = val.in[0];
            l.b = val.in[1];
            break;
        case VB200_OP_TRANSPOSE: {
            bool needed = val.keep || users[(size_t)v].empty();
            for (int u : users[(size_t)v]) needed = needed || !folds_into(v, u);
            if (!needed) continue;   // lives on only as an operand layout
            l.kind = L_TRANSPOSE;
            l.a = val.in[0];
            break;
        }
        case VB200_OP_REDUCE_SUM: case VB200_OP_REDUCE_MEAN: {
            const PValue &a = p->values[(size_t)val.in[0]];
            const int axis = (int)val.attrs[0];
            l.kind = L_REDUCE;
            l.a = val.in[0];
            // on the 2-D view (a rank-1 tensor is one row): -1 = everything, 0 = over rows, 1 = over columns
            long long reduced = a.count;
            l.axis = -1;
            if (axis >= 0 && a.shape.size() == 2) {
                l.axis = axis;
                reduced = axis == 0 ? a.R : a.C;
            }
            l.scale = val.kind == VB200_OP_REDUCE_MEAN ? 1.0f / (float)std::max<long long>(reduced, 1) : 1.0f;
            break;
        }
        case VB200_OP_MATMUL: {
            l.kind = L_GEMM;
            int a = val.in[0], b = val.in[1];
            const bool bt = p->fuse && p->values[(size_t)b].kind == VB200_OP_TRANSPOSE;
            const bool at = p->fuse && !bt && p->values[(size_t)a].kind == VB200_OP_TRANSPOSE;
            l.layout = bt ? GEMM_NT : at ? GEMM_TN : GEMM_NN;
            l.a = at ? p->values[(size_t)a].in[0] : a;
            l.b = bt ? p->values[(size_t)b].in[0] : b;
            l.m = val.R;
            l.n = val.C;
            l.k = p->values[(size_t)a].C;
            if (p->fuse && !val.keep && users[(size_t)v].size() == 1) {
                const int u = users[(size_t)v][0];
                PValue &uv = p->values[(size_t)u];
                if (uv.kind == VB200_OP_ADD && uv.shape == val.shape) {
                    // MatMul -> Add(row bias) [-> Relu | Sigmoid | Gelu]
                    const int other = uv.in[0] == v ? uv.in[1] : uv.in[0];
                    const PValue &bv = p->values[(size_t)other];
                    if (other != v && other < v && bv.R == 1 && bv.C == val.C) {
                        l.bias = other;
                        l.epi_mode = EPI_BIAS;
                        l.out = u;
                        done[(size_t)u] = 1;
                        int act_node = -1;
                        for (int w : users[(size_t)u])
                            if (act_of(p->values[(size_t)w].kind) >= 0 && act_node < 0) act_node = w;
                        if (act_node >= 0) {
                            l.epi_mode = EPI_BIAS_ACT;
                            l.epi_act = act_of(p->values[(size_t)act_node].kind);
                            l.out = act_node;
                            done[(size_t)act_node] = 1;
                            // the pre-activation is stored only when something else reads it
                            if (uv.keep || users[(size_t)u].size() > 1) l.out1 = u;
                        }
                    }
                } else if ((uv.kind == VB200_OP_RELU_BACKWARD || uv.kind == VB200_OP_GELU_BACKWARD) && uv.in[1] == v &&
                           uv.in[0] != v && uv.in[0] < v) {
                    // activation backward of a MatMul result: the GEMM's epilogue multiplies by f'(input)
                    l.epi_mode = EPI_DACT;
                    l.epi_act = uv.kind == VB200_OP_RELU_BACKWARD ? VB200_ACT_RELU : VB200_ACT_GELU;
                    l.saved = uv.in[0];
                    l.out = u;
                    done[(size_t)u] = 1;
                }
            }
            break;
        }
        default: return p->fail(VB200_ERR_UNSUPPORTED, "unsupported op kind in " + describe(val));
        }
        p->launches.push_back(l);
    }
    return VB200_OK;
}

}  // namespace

extern "C" {

vb200_program *volta_b200_program_new(void) { return new vb200_program(); }

void volta_b200_program_free(vb200_program *p) {
    if (!p) return;
    release(p);
    delete p;
}

const char *volta_b200_program_error(vb200_program *p) { return p ? p->error.c_str() : "null program"; }

int volta_b200_program_add(vb200_program *p, int32_t kind, int32_t value_id, const int32_t *inputs, int32_t n_inputs,
                           const int64_t *shape, int32_t ndim, const float *attrs, int32_t n_attrs) {
    if (!p) return VB200_ERR_INVALID;
    if (p->compiled) return p->fail(VB200_ERR_INVALID, "program_add: the program is already compiled");
    if (n_inputs < 0 || ndim < 0 || n_attrs < 0 || (n_inputs && !inputs) || (ndim && !shape) || (n_attrs && !attrs))
        return p->fail(VB200_ERR_INVALID, "program_add: bad argument");
    if (p->index_of.count(value_id)) return p->fail(VB200_ERR_INVALID, "program_add: value " + std::to_string(value_id) + " is already defined");
    PValue v;
    v.id = value_id;
    v.kind = kind;
    v.shape.assign(shape, shape + ndim);
    if (!to_2d(v.shape, &v.R, &v.C)) return p->fail(VB200_ERR_UNSUPPORTED, "tensors of rank above 2 are not supported: " + describe(v));
    v.count = v.R * v.C;
    if (v.count <= 0) return p->fail(VB200_ERR_UNSUPPORTED, "empty tensors are not supported: " + describe(v));
    for (int i = 0; i < n_inputs; ++i) {
        auto it = p->index_of.find(inputs[i]);
        if (it == p->index_of.end())
            return p->fail(VB200_ERR_INVALID, "program_add: value " + std::to_string(value_id) + " uses value " +
                                                  std::to_string(inputs[i]) + " before its definition (nodes come in schedule order)");
        v.in.push_back(it->second);
    }
    if (kind == VB200_OP_CONST) {
        if ((long long)n_attrs != v.count) return p->fail(VB200_ERR_INVALID, "ConstTensor data does not match its shape: " + describe(v));
        v.const_data.assign(attrs, attrs + n_attrs);
    } else {
        v.attrs.assign(attrs, attrs + n_attrs);
    }
    p->values.push_back(v);
    int rc = check_node(p, p->values.back());
    if (rc) {
        p->values.pop_back();
        return rc;
    }
    p->index_of[value_id] = (int)p->values.size() - 1;
    return VB200_OK;
}

int volta_b200_program_mark_output(vb200_program *p, int32_t value_id) {
    if (!p) return VB200_ERR_INVALID;
    if (p->compiled) return p->fail(VB200_ERR_INVALID, "mark_output: the program is already compiled");
    auto it = p->index_of.find(value_id);
    if (it == p->index_of.end()) return p->fail(VB200_ERR_INVALID, "mark_output: unknown value " + std::to_string(value_id));
    p->values[(size_t)it->second].keep = true;
    return VB200_OK;
}

int volta_b200_program_compile(vb200_program *p, int32_t fuse, vb200_compiled_program *info) {
    if (!p) return VB200_ERR_INVALID;
    if (p->compiled) return p->fail(VB200_ERR_INVALID, "compile: already compiled");
    if (p->attempted) return p->fail(VB200_ERR_INVALID, "compile: an earlier attempt failed; build a new program");
    if (p->values.empty()) return p->fail(VB200_ERR_INVALID, "compile: empty program");
    p->attempted = true;
    p->fuse = fuse != 0;
    const int nv = (int)p->values.size();
    // operands of Output nodes stay valid, like marked values; a kept alias keeps what it aliases
    // (users come after their operands, so one backward sweep follows every chain)
    for (int v = nv - 1; v >= 0; --v) {
        const PValue &val = p->values[(size_t)v];
        const bool alias_kind = val.kind == VB200_OP_IDENTITY || val.kind == VB200_OP_RESHAPE || val.kind == VB200_OP_OUTPUT;
        if (val.kind == VB200_OP_OUTPUT || (alias_kind && val.keep)) p->values[(size_t)val.in[0]].keep = true;
    }
    int rc = lower(p);
    if (rc) return rc;

    // ---- liveness over the launch list, then the arena
    const int end = (int)p->launches.size();
    std::vector<int> first((size_t)nv, -1), last((size_t)nv, -1);
    auto touch = [&](int v, int pos, bool write) {
        if (v < 0) return;
        const int r = p->root(v);
        if (write) {
            p->values[(size_t)r].produced = true;
            if (first[(size_t)r] < 0) first[(size_t)r] = pos;
        }
        last[(size_t)r] = std::max(last[(size_t)r], pos);
    };
    for (int pos = 0; pos < end; ++pos) {
        const Launch &l = p->launches[(size_t)pos];
        touch(l.out, pos, true);
        touch(l.out1, pos, true);
        for (int v : {l.a, l.b, l.bias, l.saved}) touch(v, pos, false);
    }
    long long red = 1, gs = 0;
    for (const Launch &l : p->launches) {
        if (l.kind == L_REDUCE) {
            const PValue &a = p->values[(size_t)l.a];
            red = std::max(red, l.axis < 0 ? loss_blocks(a.count) : colsum_chunks(a.R, a.C) * a.C);
        }
        if (l.kind == L_XENT) {
            const PValue &a = p->values[(size_t)l.a];
            red = std::max(red, a.R + loss_blocks(a.R));
        }
        if (l.kind == L_GEMM) gs = std::max(std::max(gs, ffma_scratch_floats(l.m, l.n, l.k)), gemm_tc_scratch_floats(l.layout, l.m, l.n, l.k));
    }
    ArenaPlan &pl = p->plan;
    const int i_sc = pl.add("scalars+status", 1024, 0, end, true);
    const int i_red = pl.add("reduce_scratch", red * 4, 0, end, true);
    const int i_gs = pl.add("gemm_splitk_scratch", gs * 4, 0, end, true);
    for (int v = 0; v < nv; ++v) {
        PValue &val = p->values[(size_t)v];
        if (val.alias >= 0) continue;
        if (is_source(val.kind)) {
            val.buf = pl.add("v" + std::to_string(val.id), val.count * 4, 0, end, true);
            val.produced = true;
        } else if (val.produced) {
            bool keep = val.keep;
            for (int w = 0; w < nv; ++w)
                if (p->values[(size_t)w].keep && p->root(w) == v) keep = true;
            val.buf = pl.add("v" + std::to_string(val.id), val.count * 4, first[(size_t)v], keep ? end : last[(size_t)v], keep);
        }
    }
    pl.plan();
    std::string why;
    if (!pl.verify(&why)) return p->fail(VB200_ERR_INVALID, "memory plan rejected: " + why);
    if (info) {
        info->schedule_len = nv;
        info->launches = end;
        info->peak_bytes = pl.total();
        info->unshared_bytes = pl.sum_unshared();
        // FNV-1a over the scheduled (value id, op kind, input ids) - a stable identity of the schedule, as the
        // reference's CompiledProgram.fingerprint is of its own (backend.rs:96-105; not the same hash function)
        uint64_t h = 1469598103934665603ULL;
        auto mix = [&](uint64_t x) { for (int i = 0; i < 8; ++i) { h ^= (x >> (8 * i)) & 255; h *= 1099511628211ULL; } };
        for (const PValue &v : p->values) {
            mix((uint64_t)(uint32_t)v.id);
            mix((uint64_t)(uint32_t)v.kind);
            for (int in : v.in) mix((uint64_t)(uint32_t)p->values[(size_t)in].id);
            for (int64_t d : v.shape) mix((uint64_t)d);
        }
        mix((uint64_t)pl.total());
        info->fingerprint = h;
    }

    // ---- device side
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        return p->fail(VB200_ERR_CUDA, "no CUDA device available: libvolta_b200 has no CPU fallback");
    }
    p->arena_bytes = pl.total();
    if (cudaMalloc(&p->arena, (size_t)p->arena_bytes) != cudaSuccess) {
        cudaGetLastError();
        return p->fail(VB200_ERR_OOM, "cudaMalloc of the program arena failed");
    }
    VP_CUDA(p, cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking));
    VP_CUDA(p, cudaMemsetAsync(p->arena, 0, (size_t)p->arena_bytes, p->stream));
    auto at = [&](int idx) { return reinterpret_cast<float *>(p->arena + pl.offset(idx)); };
    p->scalars = reinterpret_cast<StepScalars *>(at(i_sc));
    p->status_word = reinterpret_cast<unsigned int *>(reinterpret_cast<char *>(at(i_sc)) + 512);
    p->reduce_scratch = at(i_red);
    p->gemm_scratch = at(i_gs);
    p->gemm_scratch_floats = (long long)(pl.buffers()[(size_t)i_gs].bytes / 4);
    for (PValue &val : p->values)
        if (val.buf >= 0) {
            val.dev = at(val.buf);
            if (val.kind == VB200_OP_CONST)
                VP_CUDA(p, cudaMemcpyAsync(val.dev, val.const_data.data(), (size_t)val.count * 4, cudaMemcpyHostToDevice, p->stream));
        }
    VP_CUDA(p, cudaStreamSynchronize(p->stream));
    // every value a launch reads must exist
    for (const Launch &l : p->launches)
        for (int v : {l.a, l.b, l.bias, l.saved})
            if (v >= 0 && !p->values[(size_t)p->root(v)].dev)
                return p->fail(VB200_ERR_INVALID, "compile: " + describe(p->values[(size_t)v]) + " is read but never produced");
    if (end > 0) {
        cudaGraph_t g = nullptr;
        VP_CUDA(p, cudaStreamBeginCapture(p->stream, cudaStreamCaptureModeThreadLocal));
        rc = enqueue(p);
        cudaError_t e = cudaStreamEndCapture(p->stream, &g);
        if (rc) {
            if (g) cudaGraphDestroy(g);
            return rc;
        }
        if (e != cudaSuccess) return p->fail(VB200_ERR_CUDA, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(e));
        e = cudaGraphInstantiate(&p->graph, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) return p->fail(VB200_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
    }
    p->compiled = true;
    return VB200_OK;
}

int volta_b200_program_bind(vb200_program *p, int32_t value_id, const float *data, int64_t n) {
    if (!p || !data) return VB200_ERR_INVALID;
    if (!p->compiled) return p->fail(VB200_ERR_INVALID, "bind: compile the program first");
    auto it = p->index_of.find(value_id);
    if (it == p->index_of.end()) return p->fail(VB200_ERR_INVALID, "bind: unknown value " + std::to_string(value_id));
    PValue &v = p->values[(size_t)it->second];
    if (v.kind != VB200_OP_INPUT && v.kind != VB200_OP_PARAMETER)
        return p->fail(VB200_ERR_INVALID, "bind: " + describe(v) + " is neither an input nor a parameter");
    if (n != v.count) return p->fail(VB200_ERR_INVALID, "bind: " + describe(v) + " takes " + std::to_string(v.count) + " floats");
    cudaPointerAttributes at{};
    bool on_dev = false;
    if (cudaPointerGetAttributes(&at, data) == cudaSuccess) on_dev = at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
    else cudaGetLastError();
    VP_CUDA(p, cudaMemcpyAsync(v.dev, data, (size_t)n * 4, on_dev ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, p->stream));
    if (!on_dev) VP_CUDA(p, cudaStreamSynchronize(p->stream));   // the host buffer is borrowed for the call only
    return VB200_OK;
}

int volta_b200_program_run(vb200_program *p) {
    if (!p) return VB200_ERR_INVALID;
    if (!p->compiled) return p->fail(VB200_ERR_INVALID, "run: compile the program first");
    if (p->graph) VP_CUDA(p, cudaGraphLaunch(p->graph, p->stream));
    return VB200_OK;
}

int volta_b200_program_fetch(vb200_program *p, int32_t value_id, float *out, int64_t n) {
    if (!p || !out) return VB200_ERR_INVALID;
    if (!p->compiled) return p->fail(VB200_ERR_INVALID, "fetch: compile the program first");
    auto it = p->index_of.find(value_id);
    if (it == p->index_of.end()) return p->fail(VB200_ERR_INVALID, "fetch: unknown value " + std::to_string(value_id));
    const PValue &v = p->values[(size_t)it->second];
    const PValue &r = p->values[(size_t)p->root(it->second)];
    bool valid = is_source(r.kind) || v.keep || r.keep;
    if (!valid || !r.dev)
        return p->fail(VB200_ERR_INVALID, "fetch: " + describe(v) + " is a temporary (its storage is reused); mark it as an output before compiling");
    if (n != v.count) return p->fail(VB200_ERR_INVALID, "fetch: " + describe(v) + " holds " + std::to_string(v.count) + " floats");
    VP_CUDA(p, cudaMemcpyAsync(out, r.dev, (size_t)n * 4, cudaMemcpyDefault, p->stream));
    VP_CUDA(p, cudaStreamSynchronize(p->stream));
    unsigned int st = 0;
    VP_CUDA(p, cudaMemcpy(&st, p->status_word, sizeof st, cudaMemcpyDeviceToHost));
    if (st) return p->fail(VB200_ERR_DEVICE_WAIT, "a device-side wait gave up");
    return VB200_OK;
}

int volta_b200_program_update(vb200_program *p, const vb200_optimizer_config *cfg, const int32_t *param_ids,
                              const int32_t *grad_ids, int32_t count, uint64_t step) {
    if (!p || !cfg || count < 0 || (count && (!param_ids || !grad_ids))) return VB200_ERR_INVALID;
    if (!p->compiled) return p->fail(VB200_ERR_INVALID, "update: compile the program first");
    const int opt = cfg->optimizer;
    if (opt < VB200_OPT_SGD || opt > VB200_OPT_SGD_MOMENTUM) return p->fail(VB200_ERR_UNSUPPORTED, "update: unknown optimizer");
    StepScalars sc{};
    sc.lr = cfg->lr;
    sc.beta1 = cfg->beta1 != 0.0f ? cfg->beta1 : 0.9f;
    sc.beta2 = cfg->beta2 != 0.0f ? cfg->beta2 : 0.999f;
    sc.eps = cfg->eps != 0.0f ? cfg->eps : 1e-8f;
    sc.weight_decay = cfg->weight_decay;
    sc.momentum = cfg->momentum != 0.0f ? cfg->momentum : 0.9f;
    sc.bc1 = 1.0f - powf(sc.beta1, (float)step);
    sc.bc2 = 1.0f - powf(sc.beta2, (float)step);
    VP_CUDA(p, launch_set_scalars(p->scalars, sc, p->stream));
    const bool has1 = opt != VB200_OPT_SGD, has2 = opt == VB200_OPT_ADAM || opt == VB200_OPT_ADAMW;
    for (int i = 0; i < count; ++i) {
        auto ip = p->index_of.find(param_ids[i]), ig = p->index_of.find(grad_ids[i]);
        if (ip == p->index_of.end() || ig == p->index_of.end()) return p->fail(VB200_ERR_INVALID, "update: unknown value id");
        PValue &pv = p->values[(size_t)ip->second];
        const PValue &gv = p->values[(size_t)p->root(ig->second)];
        if (pv.kind != VB200_OP_PARAMETER) return p->fail(VB200_ERR_INVALID, "update: " + describe(pv) + " is not a parameter");
        if (gv.count != pv.count || !gv.dev || !(gv.keep || p->values[(size_t)ig->second].keep || is_source(gv.kind)))
            return p->fail(VB200_ERR_INVALID, "update: the gradient of " + describe(pv) + " must be a marked output of the same size");
        auto &st = p->opt_state[ip->second];
        if (has1 && !st.first) {
            VP_CUDA(p, cudaMalloc(&st.first, (size_t)(pv.count + 3) / 4 * 16));
            VP_CUDA(p, cudaMemsetAsync(st.first, 0, (size_t)(pv.count + 3) / 4 * 16, p->stream));
        }
        if (has2 && !st.second) {
            VP_CUDA(p, cudaMalloc(&st.second, (size_t)(pv.count + 3) / 4 * 16));
            VP_CUDA(p, cudaMemsetAsync(st.second, 0, (size_t)(pv.count + 3) / 4 * 16, p->stream));
        }
        // the runtime's AdamW decays every tensor it is given (src/engine/ir/optimizer.rs:429-441)
        VP_CUDA(p, launch_optimizer(opt, pv.dev, st.first, st.second, gv.dev, pv.count, pv.count, p->scalars, p->stream));
    }
    return VB200_OK;
}

}  // extern "C"
