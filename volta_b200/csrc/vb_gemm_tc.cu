// Tensor-core GEMM for sm_100a: tcgen05.mma (kind::tf32) with the accumulator in tensor
// memory, operands brought in by TMA, fp32 accuracy from a 3xTF32 split.
//
// Replaces the reference's three CPU GEMM families (forward sgemm, dX through
// transpose-sgemm-transpose, dW through sgemm_tn; src/engine/ir/codegen/
// mlp_train_rust_codegen.rs:310-324, 716-718, 920-929, 963, 988) and the cuBLAS call of its
// per-op CUDA backend (src/engine/ir/cuda/kernels/matmul.rs:17-118).
//
// One CTA computes one 128 x 128 tile of C = op(A) . op(B).  Per 32-deep k-block:
//   TMA warp        loads the raw fp32 A and B tiles into a 3-stage ring (mbarrier tx-count);
//   8 split warps   read a raw stage, split every value x into hi = tf32(x) and
//                   lo = tf32(x - hi) (round to nearest), and write the four tiles
//                   A_hi, A_lo, B_hi, B_lo into a 2-stage ring in the K-major 128-byte-swizzle
//                   layout the tensor core reads; operands stored with M or N contiguous
//                   (W in the forward pass, both operands of dW) are transposed on the way, so
//                   no matrix is ever transposed in global memory;
//   MMA warp        one thread issues, per 8-deep k-step, A_lo.B_hi, A_hi.B_lo and A_hi.B_hi into
//                   fp32 accumulators in TMEM, then commits the stage back to the split warps.
//                   The tensor core truncates (rounds toward zero) when it adds into an
//                   accumulator, a bias that grows with the number of additions and with the
//                   accumulator's magnitude; so the two cross terms have an accumulator of their
//                   own and A_hi.B_hi rotates over three more, and the epilogue adds the four in
//                   fp32 with round-to-nearest (measured: ~9x less error than one accumulator);
// after the last k-block the split warps become the epilogue: tcgen05.ld the accumulator
// (lane = row) and apply the fused epilogue (bias + activation, activation derivative, or a
// plain store) straight to global memory.
//
// Every wait on an mbarrier is bounded: after ~4 s without progress the CTA records a code in
// the status word, stops waiting everywhere, drains its own loads and exits normally.
#include <cuda.h>

#include <mutex>

#include "vb_common.cuh"

namespace vb {
namespace {

constexpr int BM = 128, BN = 128, BK = 32;
constexpr int RAW_STAGES = 3, MMA_STAGES = 2;
constexpr int SPLIT_WARPS = 8, SPLIT_THREADS = SPLIT_WARPS * 32;
constexpr int TMA_WARP = SPLIT_WARPS, MMA_WARP = SPLIT_WARPS + 1;
constexpr int THREADS = (SPLIT_WARPS + 2) * 32;
constexpr int TILE_BYTES = 128 * BK * 4;  // 16 KiB: one 128 x 32 fp32 operand tile
constexpr int RAW_STAGE_BYTES = 2 * TILE_BYTES;
constexpr int MMA_STAGE_BYTES = 4 * TILE_BYTES;
constexpr int SMEM_TILES = RAW_STAGES * RAW_STAGE_BYTES + MMA_STAGES * MMA_STAGE_BYTES;
constexpr int SMEM_BYTES = SMEM_TILES + 256 + 1024;  // + barriers + room to align the base to 1 KiB
constexpr int NUM_MAIN = 3;               // hi.hi accumulators, used round-robin by k-step
constexpr int TMEM_COLS = 512;            // NUM_MAIN + 1 accumulators of BN fp32 columns (all of TMEM)
constexpr int GROUP_M = 8;  // tiles are walked in bands of 8 tile rows so that a wave shares operands in L2

// status codes (which wait gave up)
constexpr unsigned ST_RAW_EMPTY = 1u, ST_RAW_FULL = 2u, ST_MMA_EMPTY = 4u, ST_MMA_FULL = 8u, ST_ACC = 16u;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait. Returns false once this or any other wait of the CTA has given up.
__device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned int *status,
                                       unsigned code) {
    if (mbar_try(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 255u) == 0u) {
            if (*abort_flag) return false;
            unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > 4000000000ull) {
                *abort_flag = 1;
                atomicOr(status, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128 bytes, groups of
// eight rows 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);  // start address
    d |= (uint64_t)(1024u >> 4) << 32;        // stride between 8-row groups
    d |= (uint64_t)1 << 46;                   // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                   // 128-byte swizzle
    return d;
}

// Instruction descriptor: D fp32, A and B tf32, both K-major, N = BN, M = BM.
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// x = hi + lo exactly: hi is x rounded to nearest tf32 (10 explicit mantissa bits; integer
// rounding on the bit pattern: add half an ulp, clear the low 13 bits), lo = x - hi is exact in
// fp32 and at most 2^-11 |x|.  The tensor core reads only the top 19 bits of each operand, so
// lo is used truncated to tf32: an error below 2^-21 |x| whose sign follows lo's, i.e. random
// with respect to x.  Three instructions per element.
template <bool LO_RN>
__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo) {
    hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
    lo = x - hi;
    if (LO_RN) lo = __uint_as_float((__float_as_uint(lo) + 0x1000u) & 0xFFFFE000u);
}

// Byte offset of element (row, 4*k4 .. 4*k4+3) inside a K-major 128-byte-swizzled tile.
__device__ __forceinline__ uint32_t swz_offset(int row, int k4) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((k4 ^ (row & 7)) << 4));
}

template <bool KMAJOR, bool LO_RN>
__device__ __forceinline__ void split_tile(const uint8_t *raw, uint8_t *hi_t, uint8_t *lo_t, int tid) {
#pragma unroll
    for (int it = 0; it < 128 * BK / 4 / SPLIT_THREADS; ++it) {
        const int item = it * SPLIT_THREADS + tid;
        float4 v;
        uint32_t off;
        if (KMAJOR) {
            // the raw tile already has the swizzled K-major layout: split in place, position by position
            off = (uint32_t)item * 16u;
            v = *reinterpret_cast<const float4 *>(raw + off);
        } else {
            // raw tile is [32 k][128 mn]: gather four k for one mn and write them as one 16-byte chunk
            const int mn = item & 127, k4 = item >> 7;
            const float *src = reinterpret_cast<const float *>(raw) + (k4 * 4) * 128 + mn;
            v = make_float4(src[0], src[128], src[256], src[384]);
            off = swz_offset(mn, k4);
        }
        float4 h, l;
        split_tf32<LO_RN>(v.x, h.x, l.x);
        split_tf32<LO_RN>(v.y, h.y, l.y);
        split_tf32<LO_RN>(v.z, h.z, l.z);
        split_tf32<LO_RN>(v.w, h.w, l.w);
        *reinterpret_cast<float4 *>(hi_t + off) = h;
        *reinterpret_cast<float4 *>(lo_t + off) = l;
    }
}

template <bool A_KMAJOR, bool B_KMAJOR, bool LO_RN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, long long M,
               long long N, long long K, int tiles_m, int tiles_n, Epilogue epi, unsigned int *status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *raw_base = smem;
    uint8_t *mma_base = smem + RAW_STAGES * RAW_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + SMEM_TILES);
    uint64_t *raw_full = bars, *raw_empty = bars + RAW_STAGES, *mma_full = bars + 2 * RAW_STAGES,
             *mma_empty = bars + 2 * RAW_STAGES + MMA_STAGES, *acc_full = bars + 2 * RAW_STAGES + 2 * MMA_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * RAW_STAGES + 2 * MMA_STAGES + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // tile coordinates: bands of GROUP_M tile rows, row index fastest inside a band
    int tm, tn;
    {
        const int t = blockIdx.x;
        const int band = t / (GROUP_M * tiles_n);
        const int first = band * GROUP_M;
        const int rows = min(GROUP_M, tiles_m - first);
        const int local = t - band * GROUP_M * tiles_n;
        tm = first + local % rows;
        tn = local / rows;
    }
    const long long m0 = (long long)tm * BM, n0 = (long long)tn * BN;
    const int kblocks = (int)((K + BK - 1) / BK);

    if (tid == 0) {
        for (int i = 0; i < RAW_STAGES; ++i) {
            mbar_init(smem_u32(&raw_full[i]), 1);
            mbar_init(smem_u32(&raw_empty[i]), SPLIT_WARPS);
        }
        for (int i = 0; i < MMA_STAGES; ++i) {
            mbar_init(smem_u32(&mma_full[i]), SPLIT_WARPS);
            mbar_init(smem_u32(&mma_empty[i]), 1);
        }
        mbar_init(smem_u32(acc_full), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == TMA_WARP) {
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < kblocks; ++kb) {
                const int r = kb % RAW_STAGES;
                const uint32_t ph = (uint32_t)((kb / RAW_STAGES) & 1);
                if (!mbar_wait(smem_u32(&raw_empty[r]), ph ^ 1u, abort_flag, status, ST_RAW_EMPTY)) break;
                const uint32_t full = smem_u32(&raw_full[r]);
                mbar_expect_tx(full, RAW_STAGE_BYTES);
                const uint32_t dst = smem_u32(raw_base + r * RAW_STAGE_BYTES);
                const int k0 = kb * BK;
                if (A_KMAJOR) tma_load_2d(dst, &map_a, full, k0, (int)m0);
                else tma_load_2d(dst, &map_a, full, (int)m0, k0);
                if (B_KMAJOR) tma_load_2d(dst + TILE_BYTES, &map_b, full, k0, (int)n0);
                else tma_load_2d(dst + TILE_BYTES, &map_b, full, (int)n0, k0);
                issued = kb + 1;
            }
            if (*abort_flag) {
                // drain: never leave the CTA while one of its own loads may still land
                for (int kb = max(0, issued - RAW_STAGES); kb < issued; ++kb) {
                    const uint32_t bar = smem_u32(&raw_full[kb % RAW_STAGES]);
                    const uint32_t ph = (uint32_t)((kb / RAW_STAGES) & 1);
                    for (int spin = 0; spin < (1 << 20) && !mbar_try(bar, ph); ++spin) {}
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < kblocks && ok; ++kb) {
                const int s = kb % MMA_STAGES;
                const uint32_t ph = (uint32_t)((kb / MMA_STAGES) & 1);
                if (!mbar_wait(smem_u32(&mma_full[s]), ph, abort_flag, status, ST_MMA_FULL)) { ok = false; break; }
                tc_fence_after();
                const uint32_t st = smem_u32(mma_base + s * MMA_STAGE_BYTES);
                const uint64_t a_hi = make_smem_desc(st), a_lo = make_smem_desc(st + TILE_BYTES),
                               b_hi = make_smem_desc(st + 2 * TILE_BYTES), b_lo = make_smem_desc(st + 3 * TILE_BYTES);
#pragma unroll
                for (int j = 0; j < BK / 8; ++j) {
                    const uint64_t adv = (uint64_t)(j * 32 >> 4);  // 8 tf32 = 32 bytes further along the swizzled row
                    const int ks = kb * (BK / 8) + j;
                    // cross terms go to their own accumulator; hi.hi rotates over NUM_MAIN accumulators
                    umma_tf32(tmem_base + NUM_MAIN * BN, a_lo + adv, b_hi + adv, ks != 0 ? 1u : 0u);
                    umma_tf32(tmem_base + NUM_MAIN * BN, a_hi + adv, b_lo + adv, 1u);
                    umma_tf32(tmem_base + (uint32_t)(ks % NUM_MAIN) * BN, a_hi + adv, b_hi + adv, ks >= NUM_MAIN ? 1u : 0u);
                }
                umma_commit(smem_u32(&mma_empty[s]));
            }
            umma_commit(smem_u32(acc_full));  // arrives when every MMA issued so far has finished
        }
    } else {
        // ---- split warps
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb) {
            const int r = kb % RAW_STAGES, s = kb % MMA_STAGES;
            const uint32_t phr = (uint32_t)((kb / RAW_STAGES) & 1), phs = (uint32_t)((kb / MMA_STAGES) & 1);
            if (!mbar_wait(smem_u32(&raw_full[r]), phr, abort_flag, status, ST_RAW_FULL)) { ok = false; break; }
            if (!mbar_wait(smem_u32(&mma_empty[s]), phs ^ 1u, abort_flag, status, ST_MMA_EMPTY)) { ok = false; break; }
            const uint8_t *raw = raw_base + r * RAW_STAGE_BYTES;
            uint8_t *st = mma_base + s * MMA_STAGE_BYTES;
            split_tile<A_KMAJOR, LO_RN>(raw, st, st + TILE_BYTES, tid);
            split_tile<B_KMAJOR, LO_RN>(raw + TILE_BYTES, st + 2 * TILE_BYTES, st + 3 * TILE_BYTES, tid);
            fence_async_smem();  // generic-proxy writes must be visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&raw_empty[r]));
                mbar_arrive(smem_u32(&mma_full[s]));
            }
        }
        // ---- epilogue
        if (ok) ok = mbar_wait(smem_u32(acc_full), 0u, abort_flag, status, ST_ACC);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            const int q = warp & 3, half = warp >> 2;
            const long long m = m0 + q * 32 + lane;
            const bool vec_ok = ((epi.ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(epi.out0) & 15) == 0) &&
                                (!epi.out1 || (reinterpret_cast<uintptr_t>(epi.out1) & 15) == 0) &&
                                (!epi.saved || (reinterpret_cast<uintptr_t>(epi.saved) & 15) == 0) &&
                                (!epi.bias || (reinterpret_cast<uintptr_t>(epi.bias) & 15) == 0);
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                const int col0 = half * 64 + c * 32;
                uint32_t v[32];
                {
                    const uint32_t t = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)col0;
                    uint32_t w[32];
                    tmem_load_32(t + NUM_MAIN * BN, v);  // cross terms first
#pragma unroll
                    for (int a = 0; a < NUM_MAIN; ++a) {
                        tmem_load_32(t + a * BN, w);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
                    }
                }
                if (m < M) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const long long n = n0 + col0 + j;
                        if (vec_ok && n + 3 < N) {
                            epi.apply4(m, n, make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                         __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])));
                        } else {
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj)
                                if (n + jj < N) epi.apply(m, n + jj, __uint_as_float(v[j + jj]));
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            cudaGetLastError();
    });
    return fn;
}

// 2-D fp32 tensor [outer x inner] (inner contiguous) read in boxes of box_outer x box_inner.
bool make_map(CUtensorMap *map, const float *base, long long inner, long long outer, int box_inner, int box_outer,
              bool swizzle128) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)inner * 4};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

int env_int(const char *name, int dflt) {
    const char *e = getenv(name);
    return e ? atoi(e) : dflt;
}

template <bool AK, bool BKM, bool LO_RN>
cudaError_t launch_one(const CUtensorMap &ma, const CUtensorMap &mb, long long m, long long n, long long k,
                       int tiles_m, int tiles_n, const Epilogue &epi, unsigned int *status, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<AK, BKM, LO_RN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    gemm_tc_kernel<AK, BKM, LO_RN><<<tiles_m * tiles_n, THREADS, SMEM_BYTES, s>>>(ma, mb, m, n, k, tiles_m, tiles_n, epi,
                                                                                 status);
    return cudaGetLastError();
}

template <bool AK, bool BKM>
cudaError_t launch_variant(const CUtensorMap &ma, const CUtensorMap &mb, long long m, long long n, long long k,
                           int tiles_m, int tiles_n, const Epilogue &epi, unsigned int *status, cudaStream_t s) {
    // VOLTA_B200_TC_LO_RN=1 also rounds the low part to tf32 explicitly (two more instructions
    // per element) instead of leaving its truncation to the tensor core.
    static const bool lo_rn = env_int("VOLTA_B200_TC_LO_RN", 0) != 0;
    if (lo_rn) return launch_one<AK, BKM, true>(ma, mb, m, n, k, tiles_m, tiles_n, epi, status, s);
    return launch_one<AK, BKM, false>(ma, mb, m, n, k, tiles_m, tiles_n, epi, status, s);
}

long long min_flops_for_tc() {
    static long long v = -1;
    if (v < 0) {
        const char *e = getenv("VOLTA_B200_TC_MIN_FLOPS");
        v = e ? atoll(e) : 0;
    }
    return v;
}

}  // namespace

// set by callers that explicitly select the CTA-pair kernel (VB200_GEMM_TENSOR_PAIR)
thread_local bool g_force_pair = false;
void gemm_tc_select_pair(bool on) { g_force_pair = on; }

bool gemm_tc_supported(int layout, const float *A, const float *B, long long m, long long n, long long k,
                       const Epilogue &epi) {
    if (m <= 0 || n <= 0 || k <= 0) return false;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) return false;
    // the contiguous extent of each operand must be a multiple of 16 bytes (TMA row pitch)
    const long long a_inner = (layout == GEMM_TN) ? m : k;
    const long long b_inner = (layout == GEMM_NT) ? k : n;
    if ((a_inner & 3) || (b_inner & 3)) return false;
    if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL) return false;
    const long long tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    if (tiles > 0x7fffffffLL) return false;
    if (2.0 * (double)m * (double)n * (double)k < (double)min_flops_for_tc()) return false;
    (void)epi;
    return encode_fn() != nullptr;
}

namespace {
bool routes_to_pair(long long m, long long n) {
    static const int version = env_int("VOLTA_B200_TC_VERSION", 3);
    const long long pair_ctas = 2 * ((m + 255) / 256) * ((n + 255) / 256);
    return m >= 256 && n >= 256 && (g_force_pair || (version == 3 && pair_ctas >= 148));
}
}  // namespace

// Split K when the output's pair tiles fill the last wave of 74 SM pairs badly (c4's dW: 256 tiles = 3.46 waves,
// a seventh of the machine idle in the fourth).  The smallest split of 2..4 that brings the waves' occupancy to
// 95 % is taken, if each split keeps at least 64 k-blocks; a function of the shape alone.
int gemm_tc_splits(int layout, long long m, long long n, long long k) {
    (void)layout;
    static const bool on = env_int("VOLTA_B200_TC_SPLITK", 1) != 0;
    if (!on || !routes_to_pair(m, n)) return 1;
    const long long tiles = ((m + 255) / 256) * ((n + 255) / 256), kblocks = (k + 31) / 32;
    const double units = 74.0;
    auto occupancy = [&](int s) { const double w = (double)(tiles * s) / units; return w / ceil(w); };
    if (occupancy(1) >= 0.95) return 1;
    for (int s = 2; s <= 4; ++s)
        if (kblocks / s >= 64 && occupancy(s) >= 0.95) return s;
    return 1;
}

long long gemm_tc_scratch_floats(int layout, long long m, long long n, long long k) {
    const int s = gemm_tc_splits(layout, m, n, k);
    return s > 1 ? (long long)s * m * n : 0;
}

cudaError_t launch_gemm_tc(int layout, const float *A, const float *B, long long m, long long n, long long k,
                           const Epilogue &epi, unsigned int *status, cudaStream_t s, float *scratch,
                           long long scratch_floats) {
    if (!gemm_tc_supported(layout, A, B, m, n, k, epi)) return cudaErrorNotSupported;
    {
        const int splits = gemm_tc_splits(layout, m, n, k);
        if (splits > 1 && scratch && scratch_floats >= (long long)splits * m * n) {
            Epilogue slab{};
            slab.mode = EPI_STORE;
            slab.out0 = scratch;
            slab.ld = n;
            cudaError_t e = launch_gemm_tc3(layout, A, B, m, n, k, slab, status, s, splits);
            if (e != cudaSuccess) return e;
            return launch_splitk_reduce(scratch, m, n, splits, epi, s);
        }
    }
    // Kernel generations: 3 = CTA-pair kernel for outputs of at least 256 x 256 (default), 2 = single-CTA
    // kernel with in-place high parts (all other shapes), 1 = the first kernel (kept for comparison).
    static const int version = env_int("VOLTA_B200_TC_VERSION", 3);
    // the pair kernel needs enough pair tiles to put a CTA on every SM, otherwise the single-CTA
    // kernel's smaller tiles spread the work better
    const long long pair_ctas = 2 * ((m + 255) / 256) * ((n + 255) / 256);
    if (m >= 256 && n >= 256 && (g_force_pair || (version == 3 && pair_ctas >= 148)))
        return launch_gemm_tc3(layout, A, B, m, n, k, epi, status, s);
    if (version >= 2) return launch_gemm_tc2(layout, A, B, m, n, k, epi, status, s);
    const bool a_kmajor = (layout != GEMM_TN), b_kmajor = (layout == GEMM_NT);
    CUtensorMap ma, mb;
    bool ok = a_kmajor ? make_map(&ma, A, k, m, BK, BM, true) : make_map(&ma, A, m, k, BM, BK, false);
    ok = ok && (b_kmajor ? make_map(&mb, B, k, n, BK, BN, true) : make_map(&mb, B, n, k, BN, BK, false));
    if (!ok) return cudaErrorNotSupported;
    const int tiles_m = (int)((m + BM - 1) / BM), tiles_n = (int)((n + BN - 1) / BN);
    if (a_kmajor && b_kmajor) return launch_variant<true, true>(ma, mb, m, n, k, tiles_m, tiles_n, epi, status, s);
    if (a_kmajor && !b_kmajor) return launch_variant<true, false>(ma, mb, m, n, k, tiles_m, tiles_n, epi, status, s);
    if (!a_kmajor && !b_kmajor) return launch_variant<false, false>(ma, mb, m, n, k, tiles_m, tiles_n, epi, status, s);
    return cudaErrorNotSupported;
}

}  // namespace vb
