// Forward GEMM for a handful of rows (single-sample and small-batch inference, the reference's
// volta_infer protocol: examples/bench_infer.c calls it 10 000 times with one row).
//
// out[rows x c] = epilogue(x[rows x r] . W[r x c]), rows <= 8.  The work is one pass over W, so
// the kernel is latency bound: what matters is how many SMs pull on W at once.  A thread-block
// cluster of S CTAs shares one 128-column slab of W and splits the r input features S ways; each
// CTA reduces its warps' partial sums in shared memory, then CTA 0 of the cluster adds the S
// partials in rank order straight out of the other CTAs' shared memory (distributed shared
// memory) and applies the epilogue.  No atomics, no scratch in HBM, no second launch; the
// summation order depends on the shape only.
#include <cooperative_groups.h>

#include "vb_common.cuh"

namespace cg = cooperative_groups;

namespace vb {

namespace {

constexpr int GV_THREADS = 256, GV_WARPS = GV_THREADS / 32, GV_COLS = 128;

template <int ROWS>
__global__ void __launch_bounds__(GV_THREADS) gemv_cluster_kernel(const float *__restrict__ x, const float *__restrict__ W,
                                                                  int rows, long long r, long long c, int k_per_cta,
                                                                  Epilogue epi) {
    extern __shared__ float sm[];
    float *xs = sm;                              // [ROWS][k_per_cta]
    // [GV_WARPS][ROWS][GV_COLS], then [ROWS][GV_COLS] CTA sums in place; written as float4, so it starts
    // on the next 16-byte boundary behind xs
    float *part = sm + (((size_t)ROWS * k_per_cta + 3) & ~(size_t)3);
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned S = cluster.num_blocks(), rank = cluster.block_rank();
    pdl_wait();
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long slab = blockIdx.x / S;
    const long long col0 = slab * GV_COLS + lane * 4;
    const long long k0 = (long long)rank * k_per_cta;
    long long k1 = k0 + k_per_cta;
    if (k1 > r) k1 = r;
    const int kk = k1 > k0 ? (int)(k1 - k0) : 0;

    for (int i = tid; i < ROWS * k_per_cta; i += GV_THREADS) {
        const int row = i / k_per_cta, k = i - row * k_per_cta;
        xs[i] = (row < rows && k < kk) ? x[(long long)row * r + k0 + k] : 0.0f;
    }
    __syncthreads();

    float4 acc[ROWS];
#pragma unroll
    for (int q = 0; q < ROWS; ++q) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col0 < c) {
        const float *wp = W + k0 * c + col0;
#pragma unroll 4
        for (int k = warp; k < kk; k += GV_WARPS) {
            const float4 w = __ldg(reinterpret_cast<const float4 *>(wp + (long long)k * c));
#pragma unroll
            for (int q = 0; q < ROWS; ++q) {
                const float xv = xs[q * k_per_cta + k];
                acc[q].x = fmaf(xv, w.x, acc[q].x);
                acc[q].y = fmaf(xv, w.y, acc[q].y);
                acc[q].z = fmaf(xv, w.z, acc[q].z);
                acc[q].w = fmaf(xv, w.w, acc[q].w);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < ROWS; ++q)
        *reinterpret_cast<float4 *>(part + ((size_t)(warp * ROWS + q) * GV_COLS + lane * 4)) = acc[q];
    __syncthreads();
    // warps in order; the CTA's sums land in warp 0's block
    for (int e = tid; e < ROWS * GV_COLS; e += GV_THREADS) {
        float t = part[e];
#pragma unroll
        for (int w = 1; w < GV_WARPS; ++w) t += part[(size_t)w * ROWS * GV_COLS + e];
        part[e] = t;  // element e of warp 0's block is read by this thread only
    }
    cluster.sync();
    if (rank == 0) {
        for (int e = tid; e < ROWS * GV_COLS; e += GV_THREADS) {
            float t = part[e];
            for (unsigned q = 1; q < S; ++q) t += cluster.map_shared_rank(part, q)[e];
            const int row = e / GV_COLS;
            const long long col = slab * GV_COLS + (e - row * GV_COLS);
            if (row < rows && col < c) epi.apply(row, col, t);
        }
    }
    cluster.sync();  // the other CTAs' shared memory must outlive the reads above
}

template <int ROWS>
cudaError_t launch_rows(const float *x, const float *W, int rows, long long r, long long c, int S, int k_per_cta,
                        const Epilogue &epi, cudaStream_t s) {
    const size_t smem = ((((size_t)ROWS * k_per_cta + 3) & ~(size_t)3) + (size_t)GV_WARPS * ROWS * GV_COLS) * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(gemv_cluster_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const long long slabs = (c + GV_COLS - 1) / GV_COLS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(slabs * S));
    cfg.blockDim = dim3(GV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)S;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, gemv_cluster_kernel<ROWS>, x, W, rows, r, c, k_per_cta, epi);
}

}  // namespace

bool gemv_rows_supported(const float *W, long long m, long long n, long long k) {
    if (m < 1 || m > 8 || n < 4 || (n & 3) || k < 32) return false;
    if (reinterpret_cast<uintptr_t>(W) & 15) return false;
    return k <= 8 * 4096;  // at most 4096 input features per CTA of the cluster (128 KiB of staged x for 8 rows)
}

cudaError_t launch_gemv_rows(const float *x, const float *W, long long m, long long n, long long k, const Epilogue &epi,
                             cudaStream_t s) {
    if (!gemv_rows_supported(W, m, n, k)) return cudaErrorNotSupported;
    // cluster size: as many CTAs (up to the portable 8) as leave each at least 32 input features
    int S = 8;
    while (S > 1 && k / S < 32) S >>= 1;
    const int k_per_cta = (int)((k + S - 1) / S);
    const int rows = (int)m;
    if (rows == 1) return launch_rows<1>(x, W, rows, k, n, S, k_per_cta, epi, s);
    if (rows == 2) return launch_rows<2>(x, W, rows, k, n, S, k_per_cta, epi, s);
    if (rows <= 4) return launch_rows<4>(x, W, rows, k, n, S, k_per_cta, epi, s);
    return launch_rows<8>(x, W, rows, k, n, S, k_per_cta, epi, s);
}

}  // namespace vb
