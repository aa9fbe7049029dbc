// Tensor-core GEMM, CTA-pair version: two CTAs of a cluster compute one 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Same contract and same ingredients as vb_gemm_tc2.cu (raw fp32 tile
// used in place as the high part, low part stored once, MN-major descriptors for operands stored
// with M or N contiguous, accumulators drained into fp32 registers every two k-blocks), but each
// CTA loads only its 128 rows of A and its 128 of the tile's 256 columns of B, and the pair's MMA
// reads both halves of B across the two SMs.  That halves the operand bytes each SM pulls out of
// L2 per flop, which is what bounds the single-CTA kernel.
//
// Per CTA: a TMA warp (plain loads into its own shared memory), 16 split warps (low parts, drain,
// epilogue: each thread keeps 64 of the CTA's 128 x 256 sums), an MMA warp.  Only the leader
// CTA (cluster rank 0) issues MMAs; the other CTA's split warps report to the leader's barriers with
// remote mbarrier arrives, and the leader's tcgen05.commit arrives on both CTAs' barriers (two
// plain commits, one per CTA).  Every mbarrier wait is bounded (~4 s).
#include <cuda.h>

#include <mutex>

#include "vb_common.cuh"

namespace vb {
namespace {

constexpr int BM = 128, BN = 256, BK = 32;  // per CTA: 128 rows x 256 columns; the pair covers 256 x 256
constexpr int RAW_STAGES = 4;   // raw tiles stay from the TMA load until the MMAs that read them retire
// Low parts stay only from the split to the same MMAs: 3 slots (with the 4 raw slots all 227 KB of shared
// memory), so that the split warps run up to two k-blocks ahead of the tensor pipe; measured 3 % faster on
// the large GEMMs than 2 slots (VOLTA_B200_TC_LO=2 selects those).
constexpr int SPLIT_WARPS = 16, SPLIT_THREADS = SPLIT_WARPS * 32;
constexpr int TMA_WARP = SPLIT_WARPS, MMA_WARP = SPLIT_WARPS + 1;
constexpr int THREADS = (SPLIT_WARPS + 2) * 32;
constexpr int TILE_BYTES = 128 * BK * 4;        // 16 KiB
constexpr int RING_BYTES = 2 * TILE_BYTES;      // one ring slot: A tile + this CTA's half of the B tile
constexpr int smem_tiles(int lo_stages) { return (RAW_STAGES + lo_stages) * RING_BYTES; }
constexpr int smem_bytes(int lo_stages) { return smem_tiles(lo_stages) + 256 + 1024; }
constexpr int TMEM_COLS = 512;                  // 2 accumulator sets x 256 columns
constexpr int DEFAULT_CHUNK = 4;                // k-blocks per accumulator drain (48 additions per accumulator)
                    // drain chunk c-1 when about to split k-block c*CHUNK + LAG
constexpr int GROUP_M = 8;

constexpr unsigned ST_STAGE_FREE = 1u, ST_RAW_FULL = 2u, ST_LO_FULL = 8u, ST_ACC_FULL = 16u, ST_ACC_EMPTY = 32u;

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
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in another CTA of the cluster.
__device__ __forceinline__ uint32_t peer_addr(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory descriptors.  K-major: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 B apart;
// a k-step (8 tf32) is 32 bytes further along the row.  MN-major (32-bit operands): 128-byte lines of
// 32 consecutive m/n per k, 128-byte swizzle with 32-byte atoms over groups of 4 k-lines (512 B);
// groups of 32 m/n are 4096 B apart (one TMA box each); a k-step is 8 lines = 1024 bytes further.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(1024u >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(4096u >> 4) << 16) | ((uint64_t)(512u >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)1 << 61);
}

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
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

__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// lo = tf32_rn(x - trunc_tf32(x)).  trunc is what the tensor core does to the raw operand; the
// remainder has at most 13 significant bits and is rounded (not truncated) to tf32's 11 so that
// its error has no preferred sign.  What is dropped altogether is lo_a * lo_b, about 1e-7 relative.
__device__ __forceinline__ float lo_part(float x) {
    float l = x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    return __uint_as_float((__float_as_uint(l) + 0x1000u) & 0xFFFFE000u);
}

__device__ __forceinline__ void split_tile(const uint8_t *raw, uint8_t *lo_t, int tid) {
#pragma unroll
    for (int it = 0; it < TILE_BYTES / 16 / SPLIT_THREADS; ++it) {
        const uint32_t off = (uint32_t)(it * SPLIT_THREADS + tid) * 16u;
        float4 v = *reinterpret_cast<const float4 *>(raw + off);
        *reinterpret_cast<float4 *>(lo_t + off) = make_float4(lo_part(v.x), lo_part(v.y), lo_part(v.z), lo_part(v.w));
    }
}

template <bool A_KMAJOR, bool B_KMAJOR, int LO_STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tc3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, long long M,
                long long N, long long K, int tiles_m, int tiles_n, Epilogue epi, unsigned int *status, int CHUNK,
                int splits) {
    extern __shared__ uint8_t smem_raw[];
    pdl_wait();   // nothing of the previous kernel's output is touched before this
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int SMEM_TILES = smem_tiles(LO_STAGES);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + SMEM_TILES);
    uint64_t *raw_full = bars, *lo_full = bars + 8, *mma_done = bars + 16, *acc_full = bars + 24, *acc_empty = bars + 26;
    uint8_t *lo_ring = smem + RAW_STAGES * RING_BYTES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 28);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();   // 0 = leader of the pair
    int tm, tn;
    {
        const int t = (int)(blockIdx.x >> 1) % (tiles_m * tiles_n);   // pair index -> tile (split-major grid)
        const int band = t / (GROUP_M * tiles_n);
        const int first = band * GROUP_M;
        const int rows = min(GROUP_M, tiles_m - first);
        const int local = t - band * GROUP_M * tiles_n;
        tm = first + local % rows;
        tn = local / rows;
    }
    // this CTA's rows of the 256-row pair tile, and its 128 of the 256 columns of B to LOAD
    const long long m0 = (long long)tm * 256 + (long long)rank * 128, n0 = (long long)tn * 256;
    const long long nb0 = n0 + (long long)rank * 128;
    // With split K, pair p works on k-blocks [kb0, kb0 + kblocks) of tile p % tiles and stores its sums as
    // slab p / tiles of the output buffer (the caller adds the slabs in order afterwards).
    const int kblocks_all = (int)((K + BK - 1) / BK);
    const int split = (int)(blockIdx.x >> 1) / (tiles_m * tiles_n);
    const int kb_per_split = (kblocks_all + splits - 1) / splits;
    const int kb0 = split * kb_per_split;
    const int kblocks = max(0, min(kb_per_split, kblocks_all - kb0));
    const int nchunks = (kblocks + CHUNK - 1) / CHUNK;

    if (tid == 0) {
        for (int i = 0; i < 8; ++i) {
            mbar_init(smem_u32(&raw_full[i]), 1);
            mbar_init(smem_u32(&lo_full[i]), 2 * SPLIT_WARPS);   // used in the leader: both CTAs' split warps
            mbar_init(smem_u32(&mma_done[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&acc_full[i]), 1);
            mbar_init(smem_u32(&acc_empty[i]), 2 * SPLIT_WARPS); // used in the leader
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers and TMEM exist before anything crosses the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == TMA_WARP) {
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < kblocks; ++kb) {
                const int s = kb % RAW_STAGES;
                const uint32_t ph = (uint32_t)((kb / RAW_STAGES) & 1);
                // slot s was last read by the MMAs of k-block kb - RAW_STAGES
                if (!mbar_wait(smem_u32(&mma_done[s]), ph ^ 1u, abort_flag, status, ST_STAGE_FREE)) break;
                const uint32_t full = smem_u32(&raw_full[s]);
                mbar_expect_tx(full, 2 * TILE_BYTES);
                const uint32_t dst = smem_u32(smem + s * RING_BYTES);
                const int k0 = (kb0 + kb) * BK;
                if (A_KMAJOR) {
                    tma_load_2d(dst, &map_a, full, k0, (int)m0);
                } else {
#pragma unroll
                    for (int g = 0; g < 4; ++g) tma_load_2d(dst + g * 4096, &map_a, full, (int)m0 + g * 32, k0);
                }
                if (B_KMAJOR) {
                    tma_load_2d(dst + TILE_BYTES, &map_b, full, k0, (int)nb0);
                } else {
#pragma unroll
                    for (int g = 0; g < 4; ++g) tma_load_2d(dst + TILE_BYTES + g * 4096, &map_b, full, (int)nb0 + g * 32, k0);
                }
                issued = kb + 1;
            }
            if (*abort_flag) {
                for (int kb = max(0, issued - RAW_STAGES); kb < issued; ++kb) {
                    const uint32_t bar = smem_u32(&raw_full[kb % RAW_STAGES]);
                    const uint32_t ph = (uint32_t)((kb / RAW_STAGES) & 1);
                    for (int spin = 0; spin < (1 << 20) && !mbar_try(bar, ph); ++spin) {}
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_KMAJOR ? 0u : 1u) << 15) |
                                   ((B_KMAJOR ? 0u : 1u) << 16) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            bool ok = true;
            for (int c = 0; c < nchunks && ok; ++c) {
                const int set = c & 1;
                if (!mbar_wait(smem_u32(&acc_empty[set]), (uint32_t)(((c >> 1) & 1) ^ 1), abort_flag, status, ST_ACC_EMPTY)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)set * 256u;
                const int kb_end = min(kblocks, (c + 1) * CHUNK);
                for (int kb = c * CHUNK; kb < kb_end; ++kb) {
                    const int s = kb % RAW_STAGES, l = kb % LO_STAGES;
                    if (!mbar_wait(smem_u32(&lo_full[l]), (uint32_t)((kb / LO_STAGES) & 1), abort_flag, status, ST_LO_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + s * RING_BYTES), sl = smem_u32(lo_ring + l * RING_BYTES);
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        const uint32_t a_off = A_KMAJOR ? (uint32_t)j * 32u : (uint32_t)j * 1024u;
                        const uint32_t b_off = B_KMAJOR ? (uint32_t)j * 32u : (uint32_t)j * 1024u;
                        const uint64_t a_hi = A_KMAJOR ? desc_kmajor(st + a_off) : desc_mnmajor(st + a_off);
                        const uint64_t a_lo = A_KMAJOR ? desc_kmajor(sl + a_off) : desc_mnmajor(sl + a_off);
                        const uint64_t b_hi = B_KMAJOR ? desc_kmajor(st + TILE_BYTES + b_off) : desc_mnmajor(st + TILE_BYTES + b_off);
                        const uint64_t b_lo = B_KMAJOR ? desc_kmajor(sl + TILE_BYTES + b_off) : desc_mnmajor(sl + TILE_BYTES + b_off);
                        const uint32_t first = (kb == c * CHUNK && j == 0) ? 0u : 1u;
                        umma_tf32(acc, a_lo, b_hi, idesc, first);   // small terms first
                        umma_tf32(acc, a_hi, b_lo, idesc, 1u);
                        umma_tf32(acc, a_hi, b_hi, idesc, 1u);
                    }
                    // both ring slots are free in BOTH CTAs once these MMAs have read them
                    umma_commit(smem_u32(&mma_done[s]));
                    umma_commit(peer_addr(smem_u32(&mma_done[s]), 1));
                }
                umma_commit(smem_u32(&acc_full[set]));
                umma_commit(peer_addr(smem_u32(&acc_full[set]), 1));
            }
        }
    } else {
        // ---- split warps: low parts, periodic accumulator drain, epilogue
        const int q = warp & 3, cg = warp >> 2;   // lane quadrant, column group of 64
        const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(cg * 64);
        const uint32_t lead_lo_full0 = peer_addr(smem_u32(&lo_full[0]), 0);
        const uint32_t lead_acc_empty0 = peer_addr(smem_u32(&acc_empty[0]), 0);
        float acc[64];
#pragma unroll
        for (int j = 0; j < 64; ++j) acc[j] = 0.0f;
        bool ok = true;
        int next_drain = 0;
        auto drain = [&](int c) -> bool {
            const int set = c & 1;
            if (!mbar_wait(smem_u32(&acc_full[set]), (uint32_t)((c >> 1) & 1), abort_flag, status, ST_ACC_FULL)) return false;
            tc_fence_after();
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                uint32_t v[16];
                tmem_load_16(t_lane + (uint32_t)set * 256u + (uint32_t)h * 16u, v);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[h * 16 + j] += __uint_as_float(v[j]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_acc_empty0 + (uint32_t)set * 8u);
            return true;
        };
        for (int kb = 0; kb < kblocks; ++kb) {
            const int s = kb % RAW_STAGES, l = kb % LO_STAGES;
            // the low-part slot was last read by the MMAs of k-block kb - LO_STAGES
            if (kb >= LO_STAGES) {
                const int j = kb - LO_STAGES;
                if (!mbar_wait(smem_u32(&mma_done[j % RAW_STAGES]), (uint32_t)((j / RAW_STAGES) & 1), abort_flag, status,
                               ST_STAGE_FREE)) {
                    ok = false;
                    break;
                }
                // ... which also means every chunk ending at or before k-block j is complete: drain it now,
                // while the MMAs work on the other accumulator set
                while (next_drain < nchunks && (next_drain + 1) * CHUNK - 1 <= j) {
                    if (!drain(next_drain)) { ok = false; break; }
                    ++next_drain;
                }
                if (!ok) break;
            }
            if (!mbar_wait(smem_u32(&raw_full[s]), (uint32_t)((kb / RAW_STAGES) & 1), abort_flag, status, ST_RAW_FULL)) {
                ok = false;
                break;
            }
            const uint8_t *st = smem + s * RING_BYTES;
            uint8_t *dl = lo_ring + l * RING_BYTES;
            split_tile(st, dl, tid);
            split_tile(st + TILE_BYTES, dl + TILE_BYTES, tid);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_lo_full0 + (uint32_t)l * 8u);
        }
        while (ok && next_drain < nchunks) {
            ok = drain(next_drain);
            ++next_drain;
        }
        if (tid == 0) pdl_trigger();   // the next kernel's CTAs may take SMs as ours retire
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            // Each thread holds one row's 64 sums.  Stored from there, a warp's float4 store would touch 32 rows
            // (32 half-used sectors); instead the warp passes its 32 x 64 block through shared memory (every ring
            // slot is idle once the last accumulator set is full: no MMA, of either CTA, reads them any more)
            // and stores two whole 256-byte row segments per instruction.
            constexpr int ST_LD = 68;   // floats per staged row: 16-byte aligned, four wavefronts per float4 write
            float *stage = reinterpret_cast<float *>(smem) + warp * (32 * ST_LD);
            if (splits > 1) epi.out0 += (long long)split * M * N;   // this pair's slab
#pragma unroll
            for (int j = 0; j < 64; j += 4)
                *reinterpret_cast<float4 *>(stage + lane * ST_LD + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
            __syncwarp();
            const bool vec_ok = ((epi.ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(epi.out0) & 15) == 0) &&
                                (!epi.out1 || (reinterpret_cast<uintptr_t>(epi.out1) & 15) == 0) &&
                                (!epi.saved || (reinterpret_cast<uintptr_t>(epi.saved) & 15) == 0) &&
                                (!epi.bias || (reinterpret_cast<uintptr_t>(epi.bias) & 15) == 0);
            const int half = lane >> 4, c4 = (lane & 15) * 4;
            const long long n = n0 + cg * 64 + c4;
#pragma unroll 4
            for (int it = 0; it < 16; ++it) {
                const int r = it * 2 + half;
                const float4 v = *reinterpret_cast<const float4 *>(stage + r * ST_LD + c4);
                const long long m = m0 + q * 32 + r;
                if (m < M) {
                    if (vec_ok && n + 3 < N) {
                        epi.apply4(m, n, v);
                    } else {
                        if (n + 0 < N) epi.apply(m, n + 0, v.x);
                        if (n + 1 < N) epi.apply(m, n + 1, v.y);
                        if (n + 2 < N) epi.apply(m, n + 2, v.z);
                        if (n + 3 < N) epi.apply(m, n + 3, v.w);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // no CTA leaves, or frees tensor memory, while its partner may still touch it
    if (warp == MMA_WARP) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn3() {
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

bool make_map3(CUtensorMap *map, const float *base, long long inner, long long outer, int box_inner, int box_outer,
               CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_fn3();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)inner * 4};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool AK, bool BKM, int LO>
cudaError_t launch3lo(const CUtensorMap &ma, const CUtensorMap &mb, long long m, long long n, long long k, int tiles_m,
                      int tiles_n, const Epilogue &epi, unsigned int *status, cudaStream_t s, int splits) {
    static bool configured[kMaxDevices] = {};
    cudaError_t e = set_smem_once(gemm_tc3_kernel<AK, BKM, LO>, smem_bytes(LO), configured);
    if (e != cudaSuccess) return e;
    static const int chunk = [] { const char *e = getenv("VOLTA_B200_TC_CHUNK"); int v = e ? atoi(e) : DEFAULT_CHUNK; return v < 2 ? 2 : (v > 16 ? 16 : v); }();
    return launch_pdl(gemm_tc3_kernel<AK, BKM, LO>, dim3(2 * tiles_m * tiles_n * splits), dim3(THREADS), smem_bytes(LO), s, ma, mb, m, n, k,
                      tiles_m, tiles_n, epi, status, chunk, splits);
}

template <bool AK, bool BKM>
cudaError_t launch3(const CUtensorMap &ma, const CUtensorMap &mb, long long m, long long n, long long k, int tiles_m,
                    int tiles_n, const Epilogue &epi, unsigned int *status, cudaStream_t s, int splits) {
    static const int lo = [] { const char *e = getenv("VOLTA_B200_TC_LO"); return (e && atoi(e) == 2) ? 2 : 3; }();
    if (lo == 3) return launch3lo<AK, BKM, 3>(ma, mb, m, n, k, tiles_m, tiles_n, epi, status, s, splits);
    return launch3lo<AK, BKM, 2>(ma, mb, m, n, k, tiles_m, tiles_n, epi, status, s, splits);
}

}  // namespace


cudaError_t launch_gemm_tc3(int layout, const float *A, const float *B, long long m, long long n, long long k,
                            const Epilogue &epi, unsigned int *status, cudaStream_t s, int splits) {
    if (splits < 1 || (splits > 1 && epi.mode != EPI_STORE)) return cudaErrorInvalidValue;
    const bool a_kmajor = (layout != GEMM_TN), b_kmajor = (layout == GEMM_NT);
    CUtensorMap ma, mb;
    bool ok = a_kmajor ? make_map3(&ma, A, k, m, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)
                       : make_map3(&ma, A, m, k, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    ok = ok && (b_kmajor ? make_map3(&mb, B, k, n, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)
                         : make_map3(&mb, B, n, k, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B));
    if (!ok) return cudaErrorNotSupported;
    const int tiles_m = (int)((m + 255) / 256), tiles_n = (int)((n + 255) / 256);  // pair tiles
    if (a_kmajor && b_kmajor) return launch3<true, true>(ma, mb, m, n, k, tiles_m, tiles_n, epi, status, s, splits);
    if (a_kmajor && !b_kmajor) return launch3<true, false>(ma, mb, m, n, k, tiles_m, tiles_n, epi, status, s, splits);
    if (!a_kmajor && !b_kmajor) return launch3<false, false>(ma, mb, m, n, k, tiles_m, tiles_n, epi, status, s, splits);
    return cudaErrorNotSupported;
}

}  // namespace vb
