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
                 long long a_sm, long long a_sk, long long b_sk, long long b_sn, Epilogue epi) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    constexpr int PAD = 4;
    __shared__ __align__(16) float As[2][BK][BM + PAD];
    __shared__ __align__(16) float Bs[2][BK][BN + PAD];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

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
            ra[j] = (gm < M && gk < K) ? __ldg(A + gm * a_sm + gk * a_sk) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < B_PER; ++j) {
            int e = tid + j * THREADS;
            int kk = b_kmajor ? (e % BK) : (e / BN);
            int nn = b_kmajor ? (e / BK) : (e % BN);
            long long gn = n0 + nn, gk = k0 + kk;
            rb[j] = (gn < N && gk < K) ? __ldg(B + gk * b_sk + gn * b_sn) : 0.0f;
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

    const long long ktiles = (K + BK - 1) / BK;
    load_tiles(0);
    store_tiles(0);
    __syncthreads();
    for (long long kt = 0; kt < ktiles; ++kt) {
        const int buf = (int)(kt & 1);
        if (kt + 1 < ktiles) load_tiles((kt + 1) * BK);
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

cudaError_t launch_gemm_ffma(int layout, const float *A, const float *B, long long m, long long n, long long k,
                             const Epilogue &epi, cudaStream_t s) {
    if (m <= 0 || n <= 0 || k <= 0) return cudaErrorInvalidValue;
    long long a_sm, a_sk, b_sk, b_sn;
    switch (layout) {
    case GEMM_NN: a_sm = k; a_sk = 1; b_sk = n; b_sn = 1; break;
    case GEMM_NT: a_sm = k; a_sk = 1; b_sk = 1; b_sn = k; break;
    case GEMM_TN: a_sm = 1; a_sk = m; b_sk = n; b_sn = 1; break;
    default: return cudaErrorInvalidValue;
    }
    // Small outputs get small tiles so that more SMs take part (the B = 64 configurations
    // are latency-bound); the choice depends on the shape only.
    long long tiles64 = ((m + 63) / 64) * ((n + 63) / 64);
    if (tiles64 >= 96 || (m >= 64 && n >= 64 && tiles64 >= 48)) {
        dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64));
        if (grid.y > 65535) return cudaErrorInvalidConfiguration;
        gemm_ffma_kernel<64, 64, 16, 4, 4><<<grid, 256, 0, s>>>(A, B, m, n, k, a_sm, a_sk, b_sk, b_sn, epi);
    } else {
        dim3 grid((unsigned)((n + 31) / 32), (unsigned)((m + 31) / 32));
        if (grid.y > 65535) return cudaErrorInvalidConfiguration;
        gemm_ffma_kernel<32, 32, 16, 4, 4><<<grid, 64, 0, s>>>(A, B, m, n, k, a_sm, a_sk, b_sk, b_sn, epi);
    }
    return cudaGetLastError();
}

}  // namespace vb
