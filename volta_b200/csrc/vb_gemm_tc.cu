// Routing of the tensor-core GEMMs (3xTF32 on tcgen05, TMA operands, TMEM accumulators).
//
// They replace the reference's three CPU GEMM families (forward sgemm, dX through
// transpose-sgemm-transpose, dW through sgemm_tn; src/engine/ir/codegen/
// mlp_train_rust_codegen.rs:310-324, 716-718, 920-929, 963, 988) and the cuBLAS call of its
// per-op CUDA backend (src/engine/ir/cuda/kernels/matmul.rs:17-118).
//
// Two kernels share one contract: gemm_tc3_kernel (vb_gemm_tc3.cu; a pair of CTAs on a 256 x 256
// tile with cta_group::2) and gemm_tc2_kernel (vb_gemm_tc2.cu; one CTA on a 128 x 128 tile).  Either
// may split K over concurrent CTAs when its tiles fill the last wave badly; the slabs are then
// added in split order by launch_splitk_reduce, which applies the epilogue.  Which kernel and how
// many splits is decided here from the shape alone (a small cost model fitted to per-k-block times
// measured on B200), so the same shape always takes the same path and sums in the same order.
#include <cuda.h>
#include <math.h>

#include <mutex>

#include "vb_common.cuh"

namespace vb {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool tensor_maps_available() {
    static bool ok = false;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess && p)
            ok = true;
        else
            cudaGetLastError();
    });
    return ok;
}

int env_int(const char *name, int dflt) {
    const char *e = getenv(name);
    return e ? atoi(e) : dflt;
}

long long min_flops_for_tc() {
    static long long v = -1;
    if (v < 0) {
        const char *e = getenv("VOLTA_B200_TC_MIN_FLOPS");
        v = e ? atoll(e) : 0;
    }
    return v;
}

struct Route {
    bool pair;   // CTA-pair kernel (else the single-CTA kernel)
    int splits;  // K splits (1 = none)
};

// Estimated time of one candidate, in microseconds.  Per 32-deep k-block a CTA pair spends ~1.8 us on
// its 256 x 256 tile and a single CTA ~1.15 us on its 128 x 128 tile (both measured under full load);
// a wave of tiles pays ~15 us / ~8 us outside its main loop (pipeline fill, accumulator drain, epilogue
// stores); split K adds one pass that reads every slab and writes the result at HBM speed.
double candidate_us(bool pair, int s, long long m, long long n, long long k) {
    const long long kblocks = (k + 31) / 32, per = (kblocks + s - 1) / s;
    const long long tiles = pair ? ((m + 255) / 256) * ((n + 255) / 256) : ((m + 127) / 128) * ((n + 127) / 128);
    const double units = pair ? 74.0 : 148.0;
    const double waves = ceil((double)(tiles * s) / units);
    double t = waves * ((double)per * (pair ? 1.8 : 1.15) + (pair ? 15.0 : 8.0));
    if (s > 1) t += 3.0 + (double)(s + 1) * (double)m * (double)n * 4.0 / 5.0e6;
    return t;
}

Route choose_route(long long m, long long n, long long k, bool force_pair, bool may_split = true) {
    static const int version = env_int("VOLTA_B200_TC_VERSION", 3);   // 2: single-CTA kernel only
    static const bool split_on = env_int("VOLTA_B200_TC_SPLITK", 1) != 0;
    const bool pair_ok = m >= 256 && n >= 256 && (force_pair || version >= 3);
    const long long kblocks = (k + 31) / 32;
    Route best{false, 1};
    double best_t = -1.0;
    // candidates in order of preference: fewer splits first, the pair kernel first; a later one must be
    // strictly faster to be taken, and by 3 % if it splits further (its slabs cost arena memory)
    for (int s = 1; s <= (split_on && may_split ? 8 : 1); ++s) {
        if (s > 1 && kblocks / s < 16) break;   // a split keeps at least 512 of K
        for (int p = pair_ok ? 1 : 0; p >= ((force_pair && pair_ok) ? 1 : 0); --p) {
            const double t = candidate_us(p != 0, s, m, n, k);
            if (best_t < 0.0 || t < best_t * (s > best.splits ? 0.97 : 1.0)) {
                best_t = t;
                best = Route{p != 0, s};
            }
        }
    }
    return best;
}

}  // namespace

bool gemm_tc_supported(int layout, const float *A, const float *B, long long m, long long n, long long k,
                       const Epilogue &epi) {
    if (m <= 0 || n <= 0 || k <= 0) return false;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) return false;
    // the contiguous extent of each operand must be a multiple of 16 bytes (TMA row pitch)
    const long long a_inner = (layout == GEMM_TN) ? m : k;
    const long long b_inner = (layout == GEMM_NT) ? k : n;
    if ((a_inner & 3) || (b_inner & 3)) return false;
    if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL) return false;
    const long long tiles = ((m + 127) / 128) * ((n + 127) / 128);
    if (tiles * 8 > 0x7fffffffLL) return false;
    if (2.0 * (double)m * (double)n * (double)k < (double)min_flops_for_tc()) return false;
    (void)epi;
    return tensor_maps_available();
}

int gemm_tc_splits(int layout, long long m, long long n, long long k, bool force_pair) {
    (void)layout;
    return choose_route(m, n, k, force_pair).splits;
}

bool gemm_tc_uses_pair(int layout, long long m, long long n, long long k, bool force_pair) {
    (void)layout;
    return choose_route(m, n, k, force_pair).pair;
}

long long gemm_tc_scratch_floats(int layout, long long m, long long n, long long k, bool force_pair) {
    const int s = gemm_tc_splits(layout, m, n, k, force_pair);
    return s > 1 ? (long long)s * m * n : 0;
}

cudaError_t launch_gemm_tc(int layout, const float *A, const float *B, long long m, long long n, long long k,
                           const Epilogue &epi, unsigned int *status, cudaStream_t s, float *scratch,
                           long long scratch_floats, bool force_pair) {
    if (!gemm_tc_supported(layout, A, B, m, n, k, epi)) return cudaErrorNotSupported;
    Route r = choose_route(m, n, k, force_pair);
    if (r.splits > 1 && !(scratch && scratch_floats >= (long long)r.splits * m * n))
        r = choose_route(m, n, k, force_pair, false);   // no room for the slabs: the best unsplit kernel
    if (r.splits > 1) {
        Epilogue slab{};
        slab.mode = EPI_STORE;
        slab.out0 = scratch;
        slab.ld = n;
        cudaError_t e = r.pair ? launch_gemm_tc3(layout, A, B, m, n, k, slab, status, s, r.splits)
                               : launch_gemm_tc2(layout, A, B, m, n, k, slab, status, s, r.splits);
        if (e != cudaSuccess) return e;
        return launch_splitk_reduce(scratch, m, n, r.splits, epi, s);
    }
    return r.pair ? launch_gemm_tc3(layout, A, B, m, n, k, epi, status, s) : launch_gemm_tc2(layout, A, B, m, n, k, epi, status, s);
}

}  // namespace vb
