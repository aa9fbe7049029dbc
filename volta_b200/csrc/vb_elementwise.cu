// Bandwidth-bound kernels of the training step: the fused optimizer update, the bias-gradient
// column reduction and the MSE loss + seed gradient.  All reductions use a fixed order and no
// atomics, so a step is bit-identical from run to run.
#include "vb_common.cuh"
#include "vb_optimizer.cuh"

namespace vb {

// ---------------------------------------------------------------------------------------
// Optimizer: one 128-bit-vectorised pass over the flat parameter region.
//
// Arithmetic follows the reference expression trees with separate roundings (the
// reference's x86 build uses AVX2 mul/add/div/sqrt without FMA,
// src/engine/ir/codegen/mlp_train_rust_codegen.rs:352-367), hence the __f*_rn intrinsics,
// which the compiler never contracts:
//   Adam/AdamW  :358-367  m = b1*m + (1-b1)*g ; v = b2*v + (1-b2)*(g*g)
//                         w = w - lr*((m/bc1)/(sqrt(v/bc2)+eps) + wd*w)
//   Adagrad     :972-977  G += g*g ; p -= lr*g/(sqrt(G)+eps)
//   SGD         :988-991  p -= lr*g
//   SGD+momentum (extension, not in the reference) v = mu*v + g ; p -= lr*v
// Weight decay applies to the first n_decay elements only (the weights; biases follow
// them in the flat layout), as the generated step decays weights but not biases (:962-966).
// ---------------------------------------------------------------------------------------
template <int OPT>
__global__ void __launch_bounds__(256) optimizer_kernel(float *__restrict__ p, float *__restrict__ s1,
                                                        float *__restrict__ s2, const float *__restrict__ g,
                                                        long long n, long long n_decay,
                                                        const StepScalars *__restrict__ scp) {
    pdl_wait();
    pdl_trigger();
    const StepScalars sc = *scp;
    constexpr bool HAS1 = (OPT != VB200_OPT_SGD);
    constexpr bool HAS2 = (OPT == VB200_OPT_ADAM || OPT == VB200_OPT_ADAMW);
    const long long n4 = n >> 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 pv = reinterpret_cast<float4 *>(p)[i];
        float4 gv = __ldcs(reinterpret_cast<const float4 *>(g) + i);
        float4 a = HAS1 ? reinterpret_cast<float4 *>(s1)[i] : make_float4(0, 0, 0, 0);
        float4 b = HAS2 ? reinterpret_cast<float4 *>(s2)[i] : make_float4(0, 0, 0, 0);
        long long e = i << 2;
        float wd0 = (OPT == VB200_OPT_ADAMW && e + 0 < n_decay) ? sc.weight_decay : 0.0f;
        float wd1 = (OPT == VB200_OPT_ADAMW && e + 1 < n_decay) ? sc.weight_decay : 0.0f;
        float wd2 = (OPT == VB200_OPT_ADAMW && e + 2 < n_decay) ? sc.weight_decay : 0.0f;
        float wd3 = (OPT == VB200_OPT_ADAMW && e + 3 < n_decay) ? sc.weight_decay : 0.0f;
        update_one<OPT>(pv.x, a.x, b.x, gv.x, sc, wd0);
        update_one<OPT>(pv.y, a.y, b.y, gv.y, sc, wd1);
        update_one<OPT>(pv.z, a.z, b.z, gv.z, sc, wd2);
        update_one<OPT>(pv.w, a.w, b.w, gv.w, sc, wd3);
        reinterpret_cast<float4 *>(p)[i] = pv;
        if (HAS1) reinterpret_cast<float4 *>(s1)[i] = a;
        if (HAS2) reinterpret_cast<float4 *>(s2)[i] = b;
    }
    // scalar tail (n not a multiple of 4): handled by the first threads of block 0
    if (blockIdx.x == 0) {
        long long e = (n4 << 2) + threadIdx.x;
        if (e < n) {
            float pv = p[e], a = HAS1 ? s1[e] : 0.0f, b = HAS2 ? s2[e] : 0.0f;
            float wd = (OPT == VB200_OPT_ADAMW && e < n_decay) ? sc.weight_decay : 0.0f;
            update_one<OPT>(pv, a, b, g[e], sc, wd);
            p[e] = pv;
            if (HAS1) s1[e] = a;
            if (HAS2) s2[e] = b;
        }
    }
}

static int sm_count() { return device_sm_count(); }

cudaError_t launch_optimizer(int optimizer, float *p, float *s1, float *s2, const float *g, long long n,
                             long long n_decay, const StepScalars *sc, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(s1) |
         reinterpret_cast<uintptr_t>(s2)) & 15)
        return cudaErrorMisalignedAddress;
    long long n4 = n >> 2;
    long long want = (n4 + 255) / 256;
    long long cap = (long long)sm_count() * 8;  // 8 resident CTAs of 256 threads per SM, grid-stride beyond
    int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    switch (optimizer) {
    case VB200_OPT_SGD: return launch_pdl(optimizer_kernel<VB200_OPT_SGD>, dim3(blocks), dim3(256), 0, s, p, s1, s2, g, n, n_decay, sc);
    case VB200_OPT_ADAM: return launch_pdl(optimizer_kernel<VB200_OPT_ADAM>, dim3(blocks), dim3(256), 0, s, p, s1, s2, g, n, n_decay, sc);
    case VB200_OPT_ADAMW: return launch_pdl(optimizer_kernel<VB200_OPT_ADAMW>, dim3(blocks), dim3(256), 0, s, p, s1, s2, g, n, n_decay, sc);
    case VB200_OPT_ADAGRAD: return launch_pdl(optimizer_kernel<VB200_OPT_ADAGRAD>, dim3(blocks), dim3(256), 0, s, p, s1, s2, g, n, n_decay, sc);
    case VB200_OPT_SGD_MOMENTUM:
        return launch_pdl(optimizer_kernel<VB200_OPT_SGD_MOMENTUM>, dim3(blocks), dim3(256), 0, s, p, s1, s2, g, n, n_decay, sc);
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// Non-finite guard.  The reference's runtime loop fails fast on a non-finite loss, gradient,
// parameter or optimizer-state element and names the first one (src/engine/ir/train.rs:670-773,
// "Non-finite {stage} {label} at element {index}"); its generated step has no such check.  One
// pass over the four flat regions finds, per region, the smallest index holding an inf or a NaN
// (all ones = none): a minimum, so the answer does not depend on the order the blocks finish in.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) finite_guard_kernel(const float *__restrict__ p, const float *__restrict__ g,
                                                           const float *__restrict__ s1, const float *__restrict__ s2,
                                                           long long n, long long n_grads,
                                                           unsigned long long *__restrict__ first_bad) {
    __shared__ unsigned long long sm[4][8];
    pdl_wait();
    pdl_trigger();
    const float *reg[4] = {g, p, s1, s2};
    unsigned long long mine[4] = {~0ULL, ~0ULL, ~0ULL, ~0ULL};
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (int r = 0; r < 4; ++r) {
        if (!reg[r]) continue;
        const long long cnt = r == 0 ? n_grads : n;   // the gradient region carries the loss sum behind it
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < cnt; i += stride) {
            const unsigned int bits = __float_as_uint(reg[r][i]);
            if ((bits & 0x7F800000u) == 0x7F800000u) { mine[r] = (unsigned long long)i; break; }
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int r = 0; r < 4; ++r) {
        unsigned long long v = mine[r];
        for (int o = 16; o; o >>= 1) {
            const unsigned long long w = __shfl_xor_sync(0xffffffffu, v, o);
            v = w < v ? w : v;
        }
        if (lane == 0) sm[r][warp] = v;
    }
    __syncthreads();
    if (threadIdx.x < 4) {
        unsigned long long v = ~0ULL;
        for (int w = 0; w < 8; ++w) v = sm[threadIdx.x][w] < v ? sm[threadIdx.x][w] : v;
        if (v != ~0ULL) atomicMin(first_bad + threadIdx.x, v);
    }
}

cudaError_t launch_finite_guard(const float *p, const float *g, const float *s1, const float *s2, long long n,
                                long long n_grads, unsigned long long *first_bad, cudaStream_t s) {
    long long want = (n + 255) / 256, cap = (long long)sm_count() * 8;
    int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    return launch_pdl(finite_guard_kernel, dim3(blocks), dim3(256), 0, s, p, g, s1, s2, n, n_grads, first_bad);
}

__global__ void set_scalars_kernel(StepScalars *dst, StepScalars v) { *dst = v; }

cudaError_t launch_set_scalars(StepScalars *dst, StepScalars v, cudaStream_t s) {
    set_scalars_kernel<<<1, 1, 0, s>>>(dst, v);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// Bias gradient: out[j] = sum_rows in[row, j]  (mlp_train_rust_codegen.rs:931-933).
// Two passes, fixed order: pass 1 sums each chunk of rows per column (8 row-lanes per
// column, combined in lane order), pass 2 adds the chunk partials in chunk order.
// ---------------------------------------------------------------------------------------
static const int CS_COLS = 128;  // columns per block (32 threads x float4)
static const int CS_TY = 8;      // row lanes per block

long long colsum_chunks(long long rows, long long cols) {
    long long col_blocks = (cols + CS_COLS - 1) / CS_COLS;
    long long target = 4LL * 148;  // aim for a few blocks per SM; depends only on the shape
    long long chunks = (target + col_blocks - 1) / col_blocks;
    long long max_chunks = (rows + 63) / 64;  // at least 64 rows per chunk
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks < 1) chunks = 1;
    if (chunks > 1024) chunks = 1024;
    return chunks;
}

__global__ void __launch_bounds__(32 * CS_TY) colsum_pass1(float *__restrict__ partial, const float *__restrict__ in,
                                                           const float *__restrict__ wgt, long long rows,
                                                           long long cols, long long rows_per_chunk) {
    __shared__ float4 sm[CS_TY][32];
    pdl_wait();
    pdl_trigger();
    const int tx = threadIdx.x, ty = threadIdx.y;
    const long long c0 = (long long)blockIdx.x * CS_COLS + tx * 4;
    const long long r0 = (long long)blockIdx.y * rows_per_chunk;
    long long r1 = r0 + rows_per_chunk;
    if (r1 > rows) r1 = rows;
    float4 acc = make_float4(0, 0, 0, 0);
    const bool vec = ((cols & 3) == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0);
    if (vec) {
        if (c0 < cols)
            for (long long r = r0 + ty; r < r1; r += CS_TY) {
                float4 v = __ldg(reinterpret_cast<const float4 *>(in + r * cols + c0));
                const float w = wgt ? wgt[r] : 1.0f;
                acc.x = fmaf(v.x, w, acc.x); acc.y = fmaf(v.y, w, acc.y);
                acc.z = fmaf(v.z, w, acc.z); acc.w = fmaf(v.w, w, acc.w);
            }
    } else {
        for (long long r = r0 + ty; r < r1; r += CS_TY) {
            const float *row = in + r * cols;
            const float w = wgt ? wgt[r] : 1.0f;
            if (c0 + 0 < cols) acc.x = fmaf(row[c0 + 0], w, acc.x);
            if (c0 + 1 < cols) acc.y = fmaf(row[c0 + 1], w, acc.y);
            if (c0 + 2 < cols) acc.z = fmaf(row[c0 + 2], w, acc.z);
            if (c0 + 3 < cols) acc.w = fmaf(row[c0 + 3], w, acc.w);
        }
    }
    sm[ty][tx] = acc;
    __syncthreads();
    if (ty == 0) {
        float4 t = sm[0][tx];
#pragma unroll
        for (int j = 1; j < CS_TY; ++j) {
            float4 v = sm[j][tx];
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
        float *dst = partial + (long long)blockIdx.y * cols;
        if (c0 + 0 < cols) dst[c0 + 0] = t.x;
        if (c0 + 1 < cols) dst[c0 + 1] = t.y;
        if (c0 + 2 < cols) dst[c0 + 2] = t.z;
        if (c0 + 3 < cols) dst[c0 + 3] = t.w;
    }
}

__global__ void colsum_pass2(float *__restrict__ out, const float *__restrict__ partial, long long chunks,
                             long long cols) {
    pdl_wait();
    pdl_trigger();
    long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float t = partial[c];
    for (long long j = 1; j < chunks; ++j) t += partial[j * cols + c];
    out[c] = t;
}

cudaError_t launch_colsum(float *out, const float *in, long long rows, long long cols, float *scratch,
                          cudaStream_t s, const float *row_weight) {
    if (rows <= 0 || cols <= 0) return cudaErrorInvalidValue;
    long long chunks = colsum_chunks(rows, cols);
    long long rpc = (rows + chunks - 1) / chunks;
    dim3 grid((unsigned)((cols + CS_COLS - 1) / CS_COLS), (unsigned)chunks), block(32, CS_TY);
    cudaError_t e = launch_pdl(colsum_pass1, grid, block, 0, s, scratch, in, row_weight, rows, cols, rpc);
    if (e != cudaSuccess) return e;
    return launch_pdl(colsum_pass2, dim3((unsigned)((cols + 255) / 256)), dim3(256), 0, s, out, (const float *)scratch, chunks, cols);
}

// ---------------------------------------------------------------------------------------
// Output layer of width one: out[row] = in[row, :] . w + bias[0].  One warp per row, each
// lane a fixed strided share of the columns, then a fixed shuffle tree.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rowdot_kernel(float *__restrict__ out, const float *__restrict__ in,
                                                     const float *__restrict__ w, const float *__restrict__ bias,
                                                     long long rows, long long cols) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    const bool vec = ((cols & 3) == 0) && (((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(w)) & 15) == 0);
    for (long long row = (((long long)blockIdx.x * blockDim.x) + threadIdx.x) >> 5; row < rows; row += warps) {
        const float *src = in + row * cols;
        float acc = 0.0f;
        if (vec) {
            for (long long c = lane * 4; c < cols; c += 128) {
                float4 a = __ldcs(reinterpret_cast<const float4 *>(src + c));
                float4 b = __ldg(reinterpret_cast<const float4 *>(w + c));
                acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
            }
        } else {
            for (long long c = lane; c < cols; c += 32) acc = fmaf(src[c], w[c], acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
        if (lane == 0) out[row] = acc + (bias ? bias[0] : 0.0f);
    }
}

cudaError_t launch_rowdot(float *out, const float *in, const float *w, const float *bias, long long rows,
                          long long cols, cudaStream_t s) {
    if (rows <= 0 || cols <= 0) return cudaErrorInvalidValue;
    long long want = (rows + 7) / 8, cap = (long long)sm_count() * 8;
    int blocks = (int)(want > cap ? cap : want);
    return launch_pdl(rowdot_kernel, dim3(blocks), dim3(256), 0, s, out, in, w, bias, rows, cols);
}

// ---------------------------------------------------------------------------------------
// dX of a width-one layer (the output layer of every benchmark model): delta . W^T with W an [r x 1]
// column is the outer product delta[row] * w[k], times the previous layer's activation derivative
// (mlp_train_rust_codegen.rs:894-929).  One streaming pass: reads `saved`, writes the result, 8 bytes per
// element, against a GEMM that would pad the single column to a tile.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rank1_dx_kernel(float *__restrict__ out, const float *__restrict__ delta,
                                                       const float *__restrict__ w, const float *__restrict__ saved, int act,
                                                       long long rows, long long cols, int vec) {
    pdl_wait();
    pdl_trigger();
    const long long stride = (long long)gridDim.x * blockDim.x, t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        const long long c4 = cols >> 2, total = rows * c4;
        for (long long i = t0; i < total; i += stride) {
            const long long row = i / c4, k = (i - row * c4) << 2;
            const float d = delta[row];
            const float4 wv = __ldg(reinterpret_cast<const float4 *>(w + k));
            float4 o = make_float4(d * wv.x, d * wv.y, d * wv.z, d * wv.w);
            if (saved) {
                const float4 sv = __ldcs(reinterpret_cast<const float4 *>(saved + row * cols + k));
                o.x *= act_backward(act, sv.x); o.y *= act_backward(act, sv.y);
                o.z *= act_backward(act, sv.z); o.w *= act_backward(act, sv.w);
            }
            *reinterpret_cast<float4 *>(out + row * cols + k) = o;
        }
    } else {
        const long long total = rows * cols;
        for (long long i = t0; i < total; i += stride) {
            const long long row = i / cols, k = i - row * cols;
            float o = delta[row] * w[k];
            if (saved) o *= act_backward(act, saved[i]);
            out[i] = o;
        }
    }
}

cudaError_t launch_rank1_dx(float *out, const float *delta, const float *w, const float *saved, int act, long long rows,
                            long long cols, cudaStream_t s) {
    if (rows <= 0 || cols <= 0) return cudaErrorInvalidValue;
    const int vec = (cols & 3) == 0 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(w) |
                                         reinterpret_cast<uintptr_t>(saved)) & 15) == 0;
    const long long work = vec ? rows * (cols >> 2) : rows * cols;
    long long want = (work + 255) / 256, cap = (long long)sm_count() * 8;
    int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    return launch_pdl(rank1_dx_kernel, dim3(blocks), dim3(256), 0, s, out, delta, w, saved, act, rows, cols, vec);
}

// ---------------------------------------------------------------------------------------
// MSE loss and seed gradient (mlp_train_rust_codegen.rs:793-798):
//   d = out - y ; delta = (2*d)/nt ; loss = (sum d*d)/nt     (division by nt on the host)
// nt is the GLOBAL element count under data parallelism, so that shard gradients add up.
// The reference sums sequentially; here each block sums 256 interleaved lanes and then a
// fixed shuffle/shared tree, and a single block adds the block partials in order.
// ---------------------------------------------------------------------------------------
static const int MSE_THREADS = 256;
static const int MSE_PER_BLOCK = 4096;

long long loss_blocks(long long nt) {
    long long b = (nt + MSE_PER_BLOCK - 1) / MSE_PER_BLOCK;
    return b < 1 ? 1 : b;
}

__device__ __forceinline__ float block_sum_256(float v, float *sm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    if (threadIdx.x == 0) {
        t = sm[0];
#pragma unroll
        for (int j = 1; j < MSE_THREADS / 32; ++j) t += sm[j];
    }
    return t;  // valid on thread 0
}

__global__ void __launch_bounds__(MSE_THREADS) mse_pass1(float *__restrict__ delta, float *__restrict__ partial,
                                                         const float *__restrict__ out, const float *__restrict__ y,
                                                         long long nt, float nt_global) {
    __shared__ float sm[MSE_THREADS / 32];
    pdl_wait();
    pdl_trigger();
    long long base = (long long)blockIdx.x * MSE_PER_BLOCK;
    float acc = 0.0f;
#pragma unroll 4
    for (int j = 0; j < MSE_PER_BLOCK / MSE_THREADS; ++j) {
        long long k = base + j * MSE_THREADS + threadIdx.x;
        if (k < nt) {
            float d = __fsub_rn(out[k], y[k]);
            acc = __fadd_rn(acc, __fmul_rn(d, d));
            delta[k] = __fdiv_rn(__fmul_rn(2.0f, d), nt_global);
        }
    }
    float t = block_sum_256(acc, sm);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

__global__ void __launch_bounds__(MSE_THREADS) mse_pass2(float *__restrict__ loss_sum,
                                                         const float *__restrict__ partial, long long nblocks) {
    __shared__ float sm[MSE_THREADS / 32];
    pdl_wait();
    pdl_trigger();
    float acc = 0.0f;
    for (long long k = threadIdx.x; k < nblocks; k += MSE_THREADS) acc += partial[k];
    float t = block_sum_256(acc, sm);
    if (threadIdx.x == 0) *loss_sum = t;
}

cudaError_t launch_mse_seed(float *delta, float *loss_sum, const float *out, const float *y, long long nt,
                            float nt_global, float *scratch, cudaStream_t s) {
    long long nb = loss_blocks(nt);
    cudaError_t e = launch_pdl(mse_pass1, dim3((unsigned)nb), dim3(MSE_THREADS), 0, s, delta, scratch, out, y, nt, nt_global);
    if (e != cudaSuccess) return e;
    return launch_pdl(mse_pass2, dim3(1), dim3(MSE_THREADS), 0, s, loss_sum, (const float *)scratch, nb);
}

// ---------------------------------------------------------------------------------------
// Self-check of update_rows (vb_optimizer.cuh: the persistent step kernel's optimizer) against
// update_one.  Group i of four elements is derived from a 64-bit mix of (seed, i): gradients and moments
// with random sign and mantissa and an exponent drawn either from the range training produces or from
// anywhere (so that groups the pre-check sends to the library path occur too), some exactly zero.
// counts[0] = elements whose p, s1 or s2 differ in any bit, [1] = groups that took the cores, [2] = groups
// that took the library path.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float operand_from(unsigned long long h, int lo, int span, bool allow_negative) {
    if ((h >> 58) == 0) return 0.0f;                                   // 1 in 64 exactly zero
    const unsigned mant = (unsigned)(h & 0x7FFFFFu);
    const unsigned ex = (unsigned)(127 + lo) + (unsigned)((h >> 23) % (unsigned)span);
    const unsigned sign = allow_negative ? (unsigned)((h >> 57) & 1u) : 0u;
    return __uint_as_float((sign << 31) | (ex << 23) | mant);
}
template <int OPT>
__global__ void __launch_bounds__(256) update_selftest_kernel(unsigned long long seed, long long groups, int wide, StepScalars sc,
                                                              unsigned long long *counts) {
    unsigned long long diff = 0, fast = 0, slow = 0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += stride) {
        float pe[4], ge[4], ae[4], be[4];
        bool ok = core_scalars_ok<OPT>(sc);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const unsigned long long h = mix64(seed + 4ULL * (unsigned long long)i + u);
            const unsigned long long h2 = mix64(h), h3 = mix64(h2), h4 = mix64(h3);
            pe[u] = operand_from(h, -8, 8, true);
            // narrow: gradients 2^-30..2^2, first moments around them, second moments around their squares
            ge[u] = wide ? operand_from(h2, -126, 253, true) : operand_from(h2, -30, 32, true);
            ae[u] = wide ? operand_from(h3, -126, 253, true) : operand_from(h3, -34, 36, true);
            be[u] = wide ? operand_from(h4, -126, 253, false) : operand_from(h4, -70, 72, false);
            ok = ok && core_operands_ok<OPT>(ae[u], be[u], ge[u], sc);
        }
        float4 p[1] = {make_float4(pe[0], pe[1], pe[2], pe[3])}, a[1] = {make_float4(ae[0], ae[1], ae[2], ae[3])},
               b[1] = {make_float4(be[0], be[1], be[2], be[3])};
        const float g[1][4] = {{ge[0], ge[1], ge[2], ge[3]}};
        update_rows<OPT, 1>(p, a, b, g, sc, sc.weight_decay);
        const float pr[4] = {p[0].x, p[0].y, p[0].z, p[0].w}, ar[4] = {a[0].x, a[0].y, a[0].z, a[0].w},
                    br[4] = {b[0].x, b[0].y, b[0].z, b[0].w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float rp = pe[u], ra = ae[u], rb = be[u];
            update_one<OPT>(rp, ra, rb, ge[u], sc, sc.weight_decay);
            const bool same = __float_as_uint(rp) == __float_as_uint(pr[u]) && __float_as_uint(ra) == __float_as_uint(ar[u]) &&
                              __float_as_uint(rb) == __float_as_uint(br[u]);
            // NaN results compare by bits too; both paths produce them through the same instructions or not at all
            diff += same ? 0 : 1;
        }
        (ok ? fast : slow) += 1;
    }
    atomicAdd(&counts[0], diff);
    atomicAdd(&counts[1], fast);
    atomicAdd(&counts[2], slow);
}

cudaError_t launch_update_selftest(int optimizer, unsigned long long seed, long long groups, int wide, const StepScalars &sc,
                                   unsigned long long *counts, cudaStream_t s) {
    const int blocks = sm_count() * 8;
    switch (optimizer) {
    case VB200_OPT_ADAM: update_selftest_kernel<VB200_OPT_ADAM><<<blocks, 256, 0, s>>>(seed, groups, wide, sc, counts); break;
    case VB200_OPT_ADAMW: update_selftest_kernel<VB200_OPT_ADAMW><<<blocks, 256, 0, s>>>(seed, groups, wide, sc, counts); break;
    case VB200_OPT_ADAGRAD: update_selftest_kernel<VB200_OPT_ADAGRAD><<<blocks, 256, 0, s>>>(seed, groups, wide, sc, counts); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace vb
