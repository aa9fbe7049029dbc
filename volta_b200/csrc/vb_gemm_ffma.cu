// FP32 FFMA GEMM with fused epilogue.  Correct for every shape and alignment; used for
// tiles too small or too ragged for the tensor-core path (the c = 1 output layer, layer
// widths that are not multiples of four) and as the reference point the tcgen05 kernel is
// checked against.  Replaces the three GEMM families of the reference's step:
//   forward  sgemm      src/engine/ir/codegen/mlp_train_rust_codegen.rs:310-314, 716-718
//   dX       transpose + sgemm + transpose                           :920-929
//   dW       sgemm_tn / sgd_fused_tn                                  :315-324, 963, 988
// Transposed operands are read through strides; nothing is transposed in memory.
// Each output element accumulates its k-products in ascending k inside one thread, so the
// result does not depend on the launch geometry.
#include "vb_common.cuh"

namespace vb {

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_ffma_kernel(const float *__restrict__ A, const float *__restrict__ B, long long M, long long N, long long K,
                 long long a_sm, long long a_sk, long long b_sk, long long b_sn, Epilogue epi, long long k_len,
                 float *__restrict__ partial) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    constexpr int PAD = 4;
    __shared__ __align__(16) float As[2][BK][BM + PAD];
    __shared__ __align__(16) float Bs[2][BK][BN + PAD];

    pdl_wait();
    pdl_trigger();
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    const long long k_lo = (long long)blockIdx.z * k_len;
    const long long k_hi = (k_lo + k_len < K) ? (k_lo + k_len) : K;
    constexpr int A_PER = BM * BK / THREADS, B_PER = BN * BK / THREADS;
    float ra[A_PER], rb[B_PER];
    const bool a_kmajor = (a_sk == 1), b_kmajor = (b_sk == 1);

    auto load_tiles = [&](long long k0) {
#pragma unroll
        for (int j = 0; j < A_PER; ++j) {
            int e = tid + j * THREADS;
            int kk = a_kmajor ? (e % BK) : (e / BM);
            int mm = a_kmajor ? (e / BK) : (e % BM);
            long long gm = m0 + mm, gk = k0 + kk;
            ra[j] = (gm < M && gk < k_hi) ? __ldg(A + gm * a_sm + gk * a_sk) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < B_PER; ++j) {
            int e = tid + j * THREADS;
            int kk = b_kmajor ? (e % BK) : (e / BN);
            int nn = b_kmajor ? (e / BK) : (e % BN);
            long long gn = n0 + nn, gk = k0 + kk;
            rb[j] = (gn < N && gk < k_hi) ? __ldg(B + gk * b_sk + gn * b_sn) : 0.0f;
        }
    };
    auto store_tiles = [&](int buf) {
#pragma unroll
        for (int j = 0; j < A_PER; ++j) {
            int e = tid + j * THREADS;
            int kk = a_kmajor ? (e % BK) : (e / BM);
            int mm = a_kmajor ? (e / BK) : (e % BM);
            As[buf][kk][mm] = ra[j];
        }
#pragma unroll
        for (int j = 0; j < B_PER; ++j) {
            int e = tid + j * THREADS;
            int kk = b_kmajor ? (e % BK) : (e / BN);
            int nn = b_kmajor ? (e / BK) : (e % BN);
            Bs[buf][kk][nn] = rb[j];
        }
    };

    // split-K: this CTA sums k in [k_lo, k_hi); with one split that is all of K
    const long long ktiles = (k_hi - k_lo + BK - 1) / BK;
    load_tiles(k_lo);
    store_tiles(0);
    __syncthreads();
    for (long long kt = 0; kt < ktiles; ++kt) {
        const int buf = (int)(kt & 1);
        if (kt + 1 < ktiles) load_tiles(k_lo + (kt + 1) * BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; i += 4) {
                float4 v = *reinterpret_cast<const float4 *>(&As[buf][kk][ty * TM + i]);
                a[i] = v.x; a[i + 1] = v.y; a[i + 2] = v.z; a[i + 3] = v.w;
            }
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                float4 v = *reinterpret_cast<const float4 *>(&Bs[buf][kk][tx * TN + j]);
                b[j] = v.x; b[j + 1] = v.y; b[j + 2] = v.z; b[j + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (kt + 1 < ktiles) {
            store_tiles(buf ^ 1);
            __syncthreads();
        }
    }

    if (partial) {
        // split-K: raw sums go to this split's slab; a second kernel adds the slabs in order
        float *dst = partial + (long long)blockIdx.z * M * N;
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            long long gm = m0 + ty * TM + i;
            if (gm >= M) continue;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                long long gn = n0 + tx * TN + j;
                if (gn < N) dst[gm * N + gn] = acc[i][j];
            }
        }
        return;
    }
    const bool vec_ok = ((epi.ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(epi.out0) & 15) == 0) &&
                        (!epi.out1 || (reinterpret_cast<uintptr_t>(epi.out1) & 15) == 0) &&
                        (!epi.saved || (reinterpret_cast<uintptr_t>(epi.saved) & 15) == 0) &&
                        (!epi.bias || (reinterpret_cast<uintptr_t>(epi.bias) & 15) == 0);
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        long long gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; j += 4) {
            long long gn = n0 + tx * TN + j;
            if (vec_ok && gn + 3 < N) {
                epi.apply4(gm, gn, make_float4(acc[i][j], acc[i][j + 1], acc[i][j + 2], acc[i][j + 3]));
            } else {
#pragma unroll
                for (int jj = 0; jj < 4; ++jj)
                    if (gn + jj < N) epi.apply(gm, gn + jj, acc[i][j + jj]);
            }
        }
    }
}

// Adds the split-K slabs in split order and applies the epilogue.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ partial, long long M, long long N,
                                                            int splits, Epilogue epi) {
    pdl_wait();
    pdl_trigger();
    const long long total = M * N;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        float v = partial[idx];
        for (int z = 1; z < splits; ++z) v += partial[(long long)z * total + idx];
        epi.apply(idx / N, idx % N, v);
    }
}

// Same for four consecutive columns (N a multiple of 4, everything 16-byte aligned).
__global__ void __launch_bounds__(256) splitk_reduce4_kernel(const float *__restrict__ partial, long long M, long long N,
                                                             int splits, Epilogue epi) {
    pdl_wait();
    pdl_trigger();
    const long long total4 = (M * N) >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
        float4 v = __ldcs(reinterpret_cast<const float4 *>(partial) + i);
        for (int z = 1; z < splits; ++z) {
            const float4 w = __ldcs(reinterpret_cast<const float4 *>(partial) + (long long)z * total4 + i);
            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        const long long idx = i << 2;
        epi.apply4(idx / N, idx % N, v);
    }
}

cudaError_t launch_splitk_reduce(const float *partial, long long m, long long n, int splits, const Epilogue &epi,
                                 cudaStream_t s) {
    const long long total = m * n;
    const bool vec = (n & 3) == 0 && (epi.ld & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(epi.out0) |
                       reinterpret_cast<uintptr_t>(epi.out1) | reinterpret_cast<uintptr_t>(epi.bias) |
                       reinterpret_cast<uintptr_t>(epi.saved)) & 15) == 0;
    if (vec) {
        const long long want = ((total >> 2) + 255) / 256;
        return launch_pdl(splitk_reduce4_kernel, dim3((unsigned)(want < 1184 ? (want < 1 ? 1 : want) : 1184)), dim3(256), 0, s, partial,
                          m, n, splits, epi);
    }
    const long long want = (total + 255) / 256;
    return launch_pdl(splitk_reduce_kernel, dim3((unsigned)(want < 1184 ? want : 1184)), dim3(256), 0, s, partial, m, n, splits, epi);
}

// How many K splits the FFMA path uses for a shape: enough CTAs to occupy the GPU when the
// output alone gives too few tiles (the batch-64 configurations), never fewer than 64 k per
// split.  A function of the shape only, so results are reproducible.
int ffma_splits(long long m, long long n, long long k) {
    const long long tiles = ((m + 63) / 64) * ((n + 63) / 64);
    if (tiles >= 96 || k < 128) return 1;
    long long want = (2 * 148 + tiles - 1) / tiles;
    long long max_by_k = k / 64;
    long long s = want < max_by_k ? want : max_by_k;
    if (s > 32) s = 32;
    return (int)(s < 1 ? 1 : s);
}

// Rough launch-time estimates (seconds) of the two GEMM paths, from measurements on B200: the
// tensor kernel pays ~8 us of fixed cost (tensor maps, TMEM, pipeline fill, epilogue) plus ~0.9 us
// per 32-deep k-block per wave of 148 tiles; the FFMA path pays ~3 us plus its flops at ~20 TFLOP/s
// scaled by how much of the GPU its CTAs cover.  Used only to route small shapes; a function of the
// shape alone.
bool gemm_prefers_tc(long long m, long long n, long long k) {
    const double flops = 2.0 * (double)m * (double)n * (double)k;
    const long long tiles128 = ((m + 127) / 128) * ((n + 127) / 128);
    const double tc = 8e-6 + (double)((tiles128 + 147) / 148) * (double)((k + 31) / 32) * 0.9e-6;
    const long long ctas = ((m + 63) / 64) * ((n + 63) / 64) * ffma_splits(m, n, k);
    const double cover = ctas >= 148 ? 1.0 : (double)ctas / 148.0;
    const double ffma = 3e-6 + flops / (20e12 * cover);
    return tc < ffma;
}

long long ffma_scratch_floats(long long m, long long n, long long k) {
    int s = ffma_splits(m, n, k);
    return s > 1 ? (long long)s * m * n : 0;
}

cudaError_t launch_gemm_ffma(int layout, const float *A, const float *B, long long m, long long n, long long k,
                             const Epilogue &epi, cudaStream_t s, float *scratch) {
    if (m <= 0 || n <= 0 || k <= 0) return cudaErrorInvalidValue;
    long long a_sm, a_sk, b_sk, b_sn;
    switch (layout) {
    case GEMM_NN: a_sm = k; a_sk = 1; b_sk = n; b_sn = 1; break;
    case GEMM_NT: a_sm = k; a_sk = 1; b_sk = 1; b_sn = k; break;
    case GEMM_TN: a_sm = 1; a_sk = m; b_sk = n; b_sn = 1; break;
    default: return cudaErrorInvalidValue;
    }
    const int splits = scratch ? ffma_splits(m, n, k) : 1;
    if (splits > 1) {
        const long long k_len = ((k + splits - 1) / splits + 15) / 16 * 16;
        const int zs = (int)((k + k_len - 1) / k_len);
        dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64), (unsigned)zs);
        cudaError_t e = launch_pdl(gemm_ffma_kernel<64, 64, 16, 4, 4>, grid, dim3(256), 0, s, A, B, m, n, k, a_sm, a_sk, b_sk, b_sn, epi, k_len, scratch);
        if (e != cudaSuccess) return e;
        long long total = m * n;
        int blocks = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
        return launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, s, (const float *)scratch, m, n, zs, epi);
    }
    // Small outputs get small tiles so that more SMs take part; the choice depends on the shape only.
    long long tiles64 = ((m + 63) / 64) * ((n + 63) / 64);
    if (tiles64 >= 96 || (m >= 64 && n >= 64 && tiles64 >= 48)) {
        dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64));
        if (grid.y > 65535) return cudaErrorInvalidConfiguration;
        return launch_pdl(gemm_ffma_kernel<64, 64, 16, 4, 4>, grid, dim3(256), 0, s, A, B, m, n, k, a_sm, a_sk, b_sk, b_sn, epi, k, (float *)nullptr);
    } else {
        dim3 grid((unsigned)((n + 31) / 32), (unsigned)((m + 31) / 32));
        if (grid.y > 65535) return cudaErrorInvalidConfiguration;
        return launch_pdl(gemm_ffma_kernel<32, 32, 16, 4, 4>, grid, dim3(64), 0, s, A, B, m, n, k, a_sm, a_sk, b_sk, b_sn, epi, k, (float *)nullptr);
    }
}

}  // namespace vb
