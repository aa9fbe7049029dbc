// Kernels of the template's optional stages, none of which a benchmark configuration uses:
// softmax as hidden activation, LayerNorm, dropout and the delta-scaling "clip"
// (src/engine/ir/codegen/mlp_train_rust_codegen.rs:727-788 forward, :829-916 backward, :936-955).
//
// Forward, a hidden layer's output runs activation -> LayerNorm -> dropout and only the final
// value is stored; backward, the delta coming out of the dX GEMM runs LayerNorm backward ->
// dropout mask -> activation backward.  Every stage needs whole rows, so one CTA takes one row,
// stages it in shared memory and applies all enabled stages in a single pass over HBM.
// Reductions use a fixed tree: a step stays bit-identical from run to run.
#include "vb_common.cuh"

namespace vb {

namespace {

constexpr int ROW_THREADS = 256;

// Sum (or max) over the CTA, the same value returned to every thread.  The butterfly gives every
// lane of a warp the same bits; the warp results are then added in warp order by every thread.
__device__ __forceinline__ float cta_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();  // the previous use of red[] is over
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int j = 1; j < ROW_THREADS / 32; ++j) t += red[j];
    return t;
}
__device__ __forceinline__ float cta_max(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int j = 1; j < ROW_THREADS / 32; ++j) t = fmaxf(t, red[j]);
    return t;
}

__global__ void __launch_bounds__(ROW_THREADS) row_forward_kernel(float *__restrict__ x, long long rows, int cols,
                                                                  RowFwd o, const StepScalars *__restrict__ sc) {
    extern __shared__ float row[];
    __shared__ float red[ROW_THREADS / 32];
    pdl_wait();
    pdl_trigger();
    const int t = threadIdx.x;
    const float fc = (float)cols;
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        float *g = x + r * cols;
        for (int j = t; j < cols; j += ROW_THREADS) row[j] = g[j];
        // each thread keeps to its own strided elements until the dropout stage, so the stages
        // below need no barrier besides the ones inside the reductions
        if (o.softmax) {  // :727-740
            float mx = -INFINITY;
            for (int j = t; j < cols; j += ROW_THREADS) mx = fmaxf(mx, row[j]);
            mx = cta_max(mx, red);
            float sum = 0.0f;
            for (int j = t; j < cols; j += ROW_THREADS) {
                float e = expf(row[j] - mx);
                row[j] = e;
                sum += e;
            }
            sum = cta_sum(sum, red);
            const float inv = 1.0f / sum;
            for (int j = t; j < cols; j += ROW_THREADS) row[j] *= inv;
        }
        if (o.ln_g) {  // :744-772
            float s = 0.0f;
            for (int j = t; j < cols; j += ROW_THREADS) s += row[j];
            const float mu = cta_sum(s, red) / fc;
            float v = 0.0f;
            for (int j = t; j < cols; j += ROW_THREADS) {
                float d = row[j] - mu;
                v += d * d;
            }
            const float var = cta_sum(v, red) / fc;
            const float is = 1.0f / sqrtf(var + 1e-5f);
            if (t == 0) o.ln_is[r] = is;
            for (int j = t; j < cols; j += ROW_THREADS) {
                float xhat = (row[j] - mu) * is;
                row[j] = __fadd_rn(__fmul_rn(xhat, o.ln_g[j]), o.ln_b[j]);
            }
        }
        if (o.dropout_p > 0.0f) {  // :773-788
            // the mask stream is sequential: every thread takes a contiguous share of the row,
            // jumps the generator to its first draw and steps from there
            __syncthreads();
            const float keep_scale = __fdiv_rn(1.0f, __fsub_rn(1.0f, o.dropout_p));   // f32 throughout, as :775
            const int chunk = (cols + ROW_THREADS - 1) / ROW_THREADS;
            const int j0 = t * chunk;
            int j1 = j0 + chunk;
            if (j1 > cols) j1 = cols;
            if (j0 < cols) {
                unsigned long long st = lcg_jump(sc->rng_base, o.draw_off + (unsigned long long)r * cols + j0);
                unsigned char *m = o.mask + r * cols;
                for (int j = j0; j < j1; ++j) {
                    st = st * kLcgA + kLcgC;
                    const float u = (float)(st >> 33) / 2147483648.0f;
                    const unsigned char keep = u >= o.dropout_p ? 1 : 0;
                    m[j] = keep;
                    row[j] = __fmul_rn(row[j], __fmul_rn((float)keep, keep_scale));
                }
            }
        }
        __syncthreads();
        for (int j = t; j < cols; j += ROW_THREADS) g[j] = row[j];
        __syncthreads();  // row[] is reused by the next row
    }
}

__global__ void __launch_bounds__(ROW_THREADS) row_backward_kernel(float *__restrict__ delta, long long rows, int cols,
                                                                   RowBwd o) {
    extern __shared__ float row[];
    __shared__ float red[ROW_THREADS / 32];
    pdl_wait();
    pdl_trigger();
    const int t = threadIdx.x;
    const float fc = (float)cols;
    const float keep_scale = o.dropout_p > 0.0f ? __fdiv_rn(1.0f, __fsub_rn(1.0f, o.dropout_p)) : 1.0f;   // f32, as :890
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        float *g = delta + r * cols;
        const float *a1 = o.a1 + r * cols;
        for (int j = t; j < cols; j += ROW_THREADS) row[j] = g[j];
        if (o.ln_g) {  // :829-887; xhat is rebuilt from the stored output, as the reference does
            const float is = o.ln_is[r];
            float sd = 0.0f, sx = 0.0f;
            for (int j = t; j < cols; j += ROW_THREADS) {
                const float gj = o.ln_g[j];
                const float xh = (a1[j] - o.ln_b[j]) / (gj + 1e-12f);
                const float dg = __fmul_rn(row[j], gj);
                sd += dg;
                sx += __fmul_rn(dg, xh);
            }
            const float sum_d = cta_sum(sd, red) / fc;
            const float sum_dxh = cta_sum(sx, red) / fc;
            for (int j = t; j < cols; j += ROW_THREADS) {
                const float gj = o.ln_g[j];
                const float xh = (a1[j] - o.ln_b[j]) / (gj + 1e-12f);
                const float d_xhat = __fmul_rn(row[j], gj);
                row[j] = __fmul_rn(is, __fsub_rn(__fsub_rn(d_xhat, sum_d), __fmul_rn(xh, sum_dxh)));
            }
        }
        if (o.dropout_p > 0.0f) {  // :888-892
            const unsigned char *m = o.mask + r * cols;
            for (int j = t; j < cols; j += ROW_THREADS) row[j] = __fmul_rn(row[j], __fmul_rn((float)m[j], keep_scale));
        }
        if (o.act == VB200_ACT_SOFTMAX) {  // :898-906
            float d = 0.0f;
            for (int j = t; j < cols; j += ROW_THREADS) d += __fmul_rn(row[j], a1[j]);
            const float dot = cta_sum(d, red);
            for (int j = t; j < cols; j += ROW_THREADS) g[j] = __fmul_rn(a1[j], __fsub_rn(row[j], dot));
        } else {  // :907-916
            const float *sv = o.saved + r * cols;
            for (int j = t; j < cols; j += ROW_THREADS) g[j] = row[j] * act_backward(o.act, sv[j]);
        }
        __syncthreads();
    }
}

// LayerNorm parameter gradients: column sums over the batch of dout*xhat and of dout, taken
// from the delta BEFORE row_backward_kernel rewrites it.  Same two-pass fixed-order scheme
// as the bias gradient.
constexpr int LG_COLS = 128, LG_TY = 8;

__global__ void __launch_bounds__(32 * LG_TY) ln_grads_pass1(float *__restrict__ partial, const float *__restrict__ dout,
                                                             const float *__restrict__ a1, const float *__restrict__ lg,
                                                             const float *__restrict__ lb, long long rows, int cols,
                                                             long long rows_per_chunk) {
    __shared__ float sg[LG_TY][LG_COLS], sb[LG_TY][LG_COLS];
    pdl_wait();
    pdl_trigger();
    const int tx = threadIdx.x, ty = threadIdx.y;
    const long long r0 = (long long)blockIdx.y * rows_per_chunk;
    long long r1 = r0 + rows_per_chunk;
    if (r1 > rows) r1 = rows;
#pragma unroll
    for (int q = 0; q < LG_COLS / 32; ++q) {
        const int c = blockIdx.x * LG_COLS + q * 32 + tx;
        float ag = 0.0f, ab = 0.0f;
        if (c < cols) {
            const float gj = lg[c] + 1e-12f, bj = lb[c];
            for (long long r = r0 + ty; r < r1; r += LG_TY) {
                const float d = dout[r * cols + c];
                const float xh = (a1[r * cols + c] - bj) / gj;
                ag = fmaf(d, xh, ag);
                ab += d;
            }
        }
        sg[ty][q * 32 + tx] = ag;
        sb[ty][q * 32 + tx] = ab;
    }
    __syncthreads();
    if (ty == 0) {
        float *dst = partial + (long long)blockIdx.y * 2 * cols;
#pragma unroll
        for (int q = 0; q < LG_COLS / 32; ++q) {
            const int c = blockIdx.x * LG_COLS + q * 32 + tx;
            if (c >= cols) continue;
            float tg = sg[0][q * 32 + tx], tb = sb[0][q * 32 + tx];
#pragma unroll
            for (int j = 1; j < LG_TY; ++j) {
                tg += sg[j][q * 32 + tx];
                tb += sb[j][q * 32 + tx];
            }
            dst[c] = tg;
            dst[cols + c] = tb;
        }
    }
}

__global__ void chunk_sum_kernel(float *__restrict__ out, const float *__restrict__ partial, long long chunks, long long n) {
    pdl_wait();
    pdl_trigger();
    long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n) return;
    float t = partial[c];
    for (long long j = 1; j < chunks; ++j) t += partial[j * n + c];
    out[c] = t;
}

// Sum of squares for the clip: 4096 elements per block, fixed tree; a single block then adds the
// block partials of all layers in order.
constexpr int SQ_THREADS = 256, SQ_PER_BLOCK = 4096;

__device__ __forceinline__ float block_sum_first(float v, float *sm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    if (threadIdx.x == 0) {
        t = sm[0];
#pragma unroll
        for (int j = 1; j < SQ_THREADS / 32; ++j) t += sm[j];
    }
    return t;  // valid on thread 0
}

__global__ void __launch_bounds__(SQ_THREADS) sumsq_kernel(float *__restrict__ partial, const float *__restrict__ v, long long n) {
    __shared__ float sm[SQ_THREADS / 32];
    pdl_wait();
    pdl_trigger();
    const long long base = (long long)blockIdx.x * SQ_PER_BLOCK;
    float acc = 0.0f;
#pragma unroll 4
    for (int j = 0; j < SQ_PER_BLOCK / SQ_THREADS; ++j) {
        long long k = base + j * SQ_THREADS + threadIdx.x;
        if (k < n) acc = fmaf(v[k], v[k], acc);
    }
    float t = block_sum_first(acc, sm);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

__global__ void __launch_bounds__(SQ_THREADS) sum_partials_kernel(float *__restrict__ out, const float *__restrict__ partial,
                                                                  long long nblocks) {
    __shared__ float sm[SQ_THREADS / 32];
    pdl_wait();
    pdl_trigger();
    float acc = 0.0f;
    for (long long k = threadIdx.x; k < nblocks; k += SQ_THREADS) acc += partial[k];
    float t = block_sum_first(acc, sm);
    if (threadIdx.x == 0) *out = t;
}

__global__ void __launch_bounds__(256) clip_scale_kernel(float *__restrict__ v, long long n, const float *__restrict__ norm_sq,
                                                         float clip) {
    pdl_wait();
    pdl_trigger();
    const float gnorm = sqrtf(*norm_sq);
    if (!(gnorm > clip)) return;  // :948-949: only ever scales down
    const float scale = clip / gnorm;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) v[i] = __fmul_rn(v[i], scale);
}

int sms() { return device_sm_count(); }

// CTAs for a one-row-per-CTA kernel with `smem` bytes each: as many as stay resident, at most one per row
int row_grid(long long rows, size_t smem) {
    long long per_sm = smem ? (long long)(200 * 1024 / smem) : 8;
    if (per_sm > 8) per_sm = 8;
    if (per_sm < 1) per_sm = 1;
    long long cap = per_sm * sms();
    return (int)(rows < cap ? rows : cap);
}

}  // namespace

cudaError_t launch_row_forward(float *x, long long rows, int cols, const RowFwd &o, const StepScalars *sc, cudaStream_t s) {
    if (rows <= 0 || cols <= 0 || cols > kRowMaxCols) return cudaErrorInvalidValue;
    const size_t smem = (size_t)cols * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(row_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    return launch_pdl(row_forward_kernel, dim3(row_grid(rows, smem)), dim3(ROW_THREADS), smem, s, x, rows, cols, o, sc);
}

cudaError_t launch_row_backward(float *delta, long long rows, int cols, const RowBwd &o, cudaStream_t s) {
    if (rows <= 0 || cols <= 0 || cols > kRowMaxCols) return cudaErrorInvalidValue;
    const size_t smem = (size_t)cols * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(row_backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    return launch_pdl(row_backward_kernel, dim3(row_grid(rows, smem)), dim3(ROW_THREADS), smem, s, delta, rows, cols, o);
}

cudaError_t launch_ln_param_grads(float *out, const float *dout, const float *a1, const float *g, const float *b,
                                  long long rows, int cols, float *scratch, cudaStream_t s) {
    if (rows <= 0 || cols <= 0) return cudaErrorInvalidValue;
    const long long chunks = colsum_chunks(rows, cols);
    const long long rpc = (rows + chunks - 1) / chunks;
    dim3 grid((unsigned)((cols + LG_COLS - 1) / LG_COLS), (unsigned)chunks), block(32, LG_TY);
    cudaError_t e = launch_pdl(ln_grads_pass1, grid, block, 0, s, scratch, dout, a1, g, b, rows, cols, rpc);
    if (e != cudaSuccess) return e;
    const long long n2 = 2LL * cols;
    return launch_pdl(chunk_sum_kernel, dim3((unsigned)((n2 + 255) / 256)), dim3(256), 0, s, out, (const float *)scratch, chunks, n2);
}

cudaError_t launch_sumsq_partials(float *partial, const float *v, long long n, cudaStream_t s) {
    if (n <= 0) return cudaErrorInvalidValue;
    return launch_pdl(sumsq_kernel, dim3((unsigned)loss_blocks(n)), dim3(SQ_THREADS), 0, s, partial, v, n);
}

cudaError_t launch_sum_partials(float *out, const float *partial, long long nblocks, cudaStream_t s) {
    return launch_pdl(sum_partials_kernel, dim3(1), dim3(SQ_THREADS), 0, s, out, partial, nblocks);
}

cudaError_t launch_clip_scale(float *v, long long n, const float *norm_sq, float clip, cudaStream_t s) {
    if (n <= 0) return cudaErrorInvalidValue;
    long long want = (n + 255) / 256, cap = (long long)sms() * 8;
    return launch_pdl(clip_scale_kernel, dim3((unsigned)(want > cap ? cap : want)), dim3(256), 0, s, v, n, norm_sq, clip);
}

}  // namespace vb
