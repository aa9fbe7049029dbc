// The whole training step as ONE persistent kernel, for batches of at most 64 rows.
//
// At batch 64 the step of the reference (src/engine/ir/codegen/mlp_train_rust_codegen.rs:699-994) is
// a chain of small dependent products whose cost on a GPU is launch and memory latency, not
// arithmetic: two dozen kernels of a few microseconds each.  Here one cooperative grid (one CTA per
// SM, grouped into thread-block clusters of S CTAs) walks the same fixed schedule
//     forward 0..n-1  ->  MSE + seed gradient  ->  backward n-1..0 (dW, db, update, dX)
// with a grid-wide barrier between phases, so that a step is one launch.
//
// Work split.  Forward layer i (act[B x r] . W[r x c]): cluster j owns a slab of output columns, its S
// CTAs split the r input features; each CTA multiplies its [B x r/S] slice by its [r/S x cols] block,
// and the S partial results are added in rank order by the CTA that owns the rows: every CTA pushes the
// rows of its partial into the owner's shared memory (distributed shared memory), the owner adds its S
// slots behind the cluster barrier and applies bias, activation, and for the last layer the loss and the
// seed gradient.  Backward layer i: cluster j owns a slab of W's ROWS, its CTAs split the columns;
// a CTA computes its block of dW = act^T . delta (the sum over the batch is local), applies the
// optimizer to exactly that block of W, m and v (streamed once), and computes its partial of
// dX = delta . W^T from the same block of (pre-update) W; the partials over the column split are
// again added in rank order through distributed shared memory, times the activation derivative.
// Bias gradients are column sums that warp 0 takes inside its product loop, spread over the clusters.
// A width-one output layer gets no phases of its own (see fuse_tail in the kernel); its per-cluster partial
// dot products (64 floats per cluster) are the only partial sums that pass through global memory, and they
// are added in cluster order.  There are no atomics on data, and every sum has a fixed order: results are
// bit-identical from run to run.
//
// One launch, nothing else: the step's scalars travel as a kernel argument, inputs that already live on
// the device are read where they lie, and CTA 0 stores the loss sum and the status word straight into
// pinned host memory, so that no copy or helper kernel surrounds the step.
//
// Memory.  Parameters and optimizer state are cold in HBM when a step starts; every CTA first asks
// for its share of the flat parameter, m and v regions to be prefetched into L2
// (cp.async.bulk.prefetch.L2), so that HBM streams them once, at full speed, underneath the forward
// phases.  Activations and deltas live in L2.  Everything another CTA wrote is read with loads that
// bypass L1 (cp.async.cg / ld.global.cg).
//
// Every wait is bounded: a grid barrier that does not complete within ~2 s sets a status bit and an
// abort word, after which no CTA waits again; the kernel then runs to its end (all cluster
// barriers are still executed) and the host reports VB200_ERR_DEVICE_WAIT.
//
// With forward_only set the kernel stops after the last layer's outputs: the reference's volta_infer
// (src/engine/ir/codegen/inner.rs:183-406) for up to 64 rows in one launch.
#include <cooperative_groups.h>

#include <type_traits>

#include "vb_common.cuh"
#include "vb_optimizer.cuh"

namespace cg = cooperative_groups;

namespace vb {
namespace {

constexpr int T = 256;          // threads per CTA
constexpr int BM = 64;          // rows of the batch at most
constexpr int KT = 128;         // depth of one staged tile (input features forward, columns backward)
constexpr int LD = KT + 4;      // shared-memory pitch of a [.. x KT] tile (conflict-free float4 reads)
constexpr int WMAX = 64;        // widest slab of W one cluster owns (columns forward, rows backward)
constexpr int LDW = WMAX + 4;   // pitch of a [.. x WMAX] tile
constexpr int BUF_A = BM * LD;          // activation / delta tile [BM][LD]
constexpr int BUF_B = KT * LDW;         // W tile: forward [KT][LDW]; backward [WMAX][LD] (8448 <= 8704)
constexpr int PART = T * 16;            // every thread's 4 x 4 partial sums
constexpr int RECV = BM * WMAX;          // the cluster's partials of this CTA's rows: [S][BM / S][<= WMAX]
constexpr int SMEM_FLOATS = 2 * BUF_A + 2 * BUF_B + BM * LDW + PART + RECV + 64;
constexpr unsigned ST_GRID_BARRIER = 128u;


__device__ __forceinline__ int round4(int v) { return (v + 3) & ~3; }
__device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

__device__ __forceinline__ void cp_async16(float *dst_smem, const float *src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
// A streaming 16-byte load that stays where it is written: the compiler neither sinks it towards its first
// use nor merges it with others, so a load placed ahead of a long computation really is in flight during it.
__device__ __forceinline__ float4 load_early(const float *p) {
    float4 v;
    asm volatile("ld.global.cs.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// dst[rows_pad x cols_pad] (pitch dst_ld) = src[rows x cols] (pitch src_ld), zero beyond rows/cols.
// 16-byte asynchronous copies when the source allows it (the caller commits and waits), plain L2 loads
// otherwise.  cols_pad is a multiple of 4.
__device__ __forceinline__ void load_tile(float *dst, int dst_ld, const float *src, long long src_ld, int rows, int cols,
                                          int rows_pad, int cols_pad) {
    const bool vec = ((src_ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && ((cols & 3) == 0);
    if (vec) {
        const int cpr = cols_pad >> 2;
        for (int idx = threadIdx.x; idx < rows_pad * cpr; idx += T) {
            const int rr = idx / cpr, cc = (idx - rr * cpr) << 2;
            const bool ok = rr < rows && cc < cols;
            cp_async16(dst + rr * dst_ld + cc, ok ? src + (long long)rr * src_ld + cc : src, ok);
        }
    } else {
        // groups of four destination floats, each element loaded on its own where it exists; rows run fastest
        // over the threads, so that the few groups of a one-column operand that hold data go to different threads
        const int cpr = cols_pad >> 2;
        for (int idx = threadIdx.x; idx < rows_pad * cpr; idx += T) {
            const int gg = idx / rows_pad, rr = idx - gg * rows_pad, cc = gg << 2;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (rr < rows && cc < cols) {
                const float *p = src + (long long)rr * src_ld + cc;
                v.x = __ldcg(p);
                if (cc + 1 < cols) v.y = __ldcg(p + 1);
                if (cc + 2 < cols) v.z = __ldcg(p + 2);
                if (cc + 3 < cols) v.w = __ldcg(p + 3);
            }
            *reinterpret_cast<float4 *>(dst + rr * dst_ld + cc) = v;
        }
    }
}

struct Barrier {
    unsigned *count, *abort_word, *status;
    unsigned phase;   // top bit of *count as of the last barrier this CTA passed (thread 0's copy is the one used)
};

// Grid-wide barrier on ONE word: CTA 0 adds 2^31 - (G - 1), every other CTA adds 1, so the word's top bit
// flips exactly when all G have arrived (and its low bits are back where they were: no reset, no second
// word).  Per CTA one fire-and-forget reduction, then a spin on the same word until its top bit differs from
// the phase the CTA remembers (read once at kernel start: the bit cannot flip before this CTA's own first
// arrival), so that an arrival costs no round trip of its own.  Bounded: after ~2 s without release the CTA
// records the failure in the status word and raises the abort word, which every spinning CTA looks at now
// and then; from there on the barriers of this launch fall through after a few hundred polls.
__device__ __forceinline__ void grid_barrier(Barrier &b) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned inc = blockIdx.x == 0 ? 0x80000000u - (gridDim.x - 1u) : 1u;
        asm volatile("red.global.add.u32 [%0], %1;" ::"l"(b.count), "r"(inc) : "memory");
        const unsigned before = b.phase;
        unsigned long long t0 = 0;
        for (unsigned it = 0;; ++it) {
            if (((*reinterpret_cast<volatile unsigned *>(b.count)) & 0x80000000u) != before) break;
            if ((it & 255u) == 255u) {
                if (*reinterpret_cast<volatile unsigned *>(b.abort_word) != 0u) break;
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                if (now - t0 > 2000000000ull) {
                    atomicOr(b.status, ST_GRID_BARRIER);
                    atomicExch(b.abort_word, 1u);
                    break;
                }
            }
        }
        b.phase = before ^ 0x80000000u;
        __threadfence();
    }
    __syncthreads();
}

// 4 x 4 register tile: acc[i][j] += sum_u a[i].u * w[u].j  (forward: a along k, w rows k..k+3)
__device__ __forceinline__ void fma_nn(float (&acc)[4][4], const float4 (&a)[4], const float4 (&w)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc[i][0] = fmaf(a[i].x, w[0].x, acc[i][0]); acc[i][1] = fmaf(a[i].x, w[0].y, acc[i][1]);
        acc[i][2] = fmaf(a[i].x, w[0].z, acc[i][2]); acc[i][3] = fmaf(a[i].x, w[0].w, acc[i][3]);
        acc[i][0] = fmaf(a[i].y, w[1].x, acc[i][0]); acc[i][1] = fmaf(a[i].y, w[1].y, acc[i][1]);
        acc[i][2] = fmaf(a[i].y, w[1].z, acc[i][2]); acc[i][3] = fmaf(a[i].y, w[1].w, acc[i][3]);
        acc[i][0] = fmaf(a[i].z, w[2].x, acc[i][0]); acc[i][1] = fmaf(a[i].z, w[2].y, acc[i][1]);
        acc[i][2] = fmaf(a[i].z, w[2].z, acc[i][2]); acc[i][3] = fmaf(a[i].z, w[2].w, acc[i][3]);
        acc[i][0] = fmaf(a[i].w, w[3].x, acc[i][0]); acc[i][1] = fmaf(a[i].w, w[3].y, acc[i][1]);
        acc[i][2] = fmaf(a[i].w, w[3].z, acc[i][2]); acc[i][3] = fmaf(a[i].w, w[3].w, acc[i][3]);
    }
}
// acc[i][j] += a[i] . w[j]  (both along the reduction dimension)
__device__ __forceinline__ void fma_nt(float (&acc)[4][4], const float4 (&a)[4], const float4 (&w)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = fmaf(a[i].x, w[j].x, acc[i][j]);
            acc[i][j] = fmaf(a[i].y, w[j].y, acc[i][j]);
            acc[i][j] = fmaf(a[i].z, w[j].z, acc[i][j]);
            acc[i][j] = fmaf(a[i].w, w[j].w, acc[i][j]);
        }
}

// How the 256 threads cover a [64 x 4*CG] result in 4 x 4 register tiles, KG of them sharing each tile
// and splitting the reduction range.  Within a warp 8 row groups x 4 column groups, which keeps every
// float4 read of the operand tiles free of bank conflicts.
struct TileMap {
    int CG, KG, kg, rg, cg;
    bool active;
};
__device__ __forceinline__ TileMap tile_map(int width) {
    TileMap m;
    m.CG = ((width + 3) / 4 + 3) & ~3;       // column groups, a multiple of 4 (4..16)
    const int t_out = 16 * m.CG;
    m.KG = T / t_out;                        // 4, 2, 1, 1
    m.kg = threadIdx.x / t_out;
    m.active = m.kg < m.KG;
    const int local = threadIdx.x - m.kg * t_out, lane = local & 31, wq = local >> 5;
    m.rg = (lane & 7) + 8 * (wq & 1);
    m.cg = (lane >> 3) + 4 * (wq >> 1);
    return m;
}

// The KG partial tiles of this CTA, part[kg][row][col], are summed in k-group order and every row of the sum is
// PUSHED into the shared memory of the CTA that owns the row (rows RB*o .. RB*o + RB - 1 belong to rank o), into
// this rank's slot there: recv[rank][row - RB*o][col].  After the cluster barrier that follows, an owner finds all
// S ranks' partials of its rows in its own shared memory (no remote read on the critical path).
__device__ __forceinline__ void fold_and_push(cg::cluster_group &cluster, const float *part, float *recv, int KG, int PLD, int S,
                                              int q) {
    __syncthreads();
    const int RB = BM / S, n4 = (BM * PLD) >> 2, p4 = PLD >> 2;
    for (int e = threadIdx.x; e < n4; e += T) {
        float4 v = reinterpret_cast<const float4 *>(part)[e];
        for (int g = 1; g < KG; ++g) {
            const float4 w = reinterpret_cast<const float4 *>(part + g * BM * PLD)[e];
            v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        const int row = e / p4, c4 = e - row * p4, owner = row / RB, rl = row - owner * RB;
        float *dst = cluster.map_shared_rank(recv, owner) + ((q * RB + rl) * PLD + (c4 << 2));
        *reinterpret_cast<float4 *>(dst) = v;
    }
}
// Element (row_local, col) of the S ranks' partials in this CTA's receive slots, added in rank order.
__device__ __forceinline__ float sum_ranks(const float *recv, int S, int RB, int PLD, int row_local, int col) {
    float v[8];
#pragma unroll
    for (int p = 0; p < 8; ++p) v[p] = p < S ? recv[((p * RB) + row_local) * PLD + col] : 0.0f;
    float sum = v[0];
#pragma unroll
    for (int p = 1; p < 8; ++p)
        if (p < S) sum += v[p];
    return sum;
}

// (Kept out of line: the measurement protocol flushes the L2 between steps, which also evicts the kernel's code,
// so every instruction executed for the first time in a step is fetched from HBM; this rarely taken path is
// inlined nowhere.)
template <int OPT>
__device__ __noinline__ void update_elem_call(float *p, float *s1, float *s2, float *gout, float g, float lr, float beta1,
                                              float beta2, float eps, float bc1, float bc2, float momentum, float wd) {
    constexpr bool HAS1 = (OPT != VB200_OPT_SGD);
    constexpr bool HAS2 = (OPT == VB200_OPT_ADAM || OPT == VB200_OPT_ADAMW);
    StepScalars sc{};
    sc.lr = lr; sc.beta1 = beta1; sc.beta2 = beta2; sc.eps = eps; sc.bc1 = bc1; sc.bc2 = bc2; sc.momentum = momentum;
    float pv = *p, a = HAS1 ? __ldcs(s1) : 0.0f, b = HAS2 ? __ldcs(s2) : 0.0f;
    update_one<OPT>(pv, a, b, g, sc, wd);
    *p = pv;
    if (HAS1) *s1 = a;
    if (HAS2) *s2 = b;
    *gout = g;
}
template <int OPT>
__device__ __forceinline__ void update_elem(float *p, float *s1, float *s2, float *gout, float g, const StepScalars &sc,
                                            float wd) {
    update_elem_call<OPT>(p, s1, s2, gout, g, sc.lr, sc.beta1, sc.beta2, sc.eps, sc.bc1, sc.bc2, sc.momentum, wd);
}

template <int OPT>
__global__ void __launch_bounds__(T, 1) small_step_kernel(const __grid_constant__ SmallStepArgs A) {
    extern __shared__ __align__(16) float smem[];
    float *bufA = smem;                        // [2][BUF_A]
    float *bufB = bufA + 2 * BUF_A;            // [2][BUF_B]
    float *actc = bufB + 2 * BUF_B;            // backward: act slice [BM][LDW]
    float *part = actc + BM * LDW;             // [PART]
    float *recv = part + PART;                 // [RECV]
    float *red = recv + RECV;                  // [64]

    cg::cluster_group cluster = cg::this_cluster();
    const int S = (int)cluster.num_blocks(), q = (int)cluster.block_rank();
    const int NC = (int)gridDim.x / S, j = (int)blockIdx.x / S;
    const int tid = threadIdx.x, B = A.B, n = A.n;
    const int RB = BM / S;                     // rows whose partials this CTA adds up

    Barrier bar;
    bar.count = A.barrier;
    bar.abort_word = A.barrier + 2;
    bar.status = A.status;
    bar.phase = tid == 0 ? (*reinterpret_cast<volatile unsigned *>(A.barrier) & 0x80000000u) : 0u;

    // ---- ask for this CTA's share of parameters and optimizer state to be brought into L2
    if (tid < 3) {
        const float *base = tid == 0 ? A.params : (tid == 1 ? A.s1 : A.s2);
        const bool wanted = tid == 0 || (tid == 1 && OPT != VB200_OPT_SGD) || (tid == 2 && (OPT == VB200_OPT_ADAM || OPT == VB200_OPT_ADAMW));
        if (wanted && base) {
            const long long total = A.n_params_padded * 4LL;                       // bytes, a multiple of 256
            const long long per = ((total + gridDim.x - 1) / gridDim.x + 255) & ~255LL;
            long long lo = per * blockIdx.x, hi = lo + per < total ? lo + per : total;
            for (; lo < hi; lo += 16384) {
                const unsigned sz = (unsigned)(hi - lo < 16384 ? hi - lo : 16384);
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<const char *>(base) + lo), "r"(sz) : "memory");
            }
        }
    }
    const StepScalars &sc = A.scalars;

    // A width-one output layer (every regression head) is not given phases of its own: its forward is a dot
    // product per row, which the clusters take over their slabs of the last hidden layer while they still hold
    // them (partials to zpart, summed in cluster order behind the next grid barrier by whoever needs the
    // result), and its backward is elementwise in dX and a 64-term sum per weight, which the tail phase below
    // does without tiles, shared-memory reductions or cluster barriers.  Two grid phases less per step.
    const bool fuse_tail = n >= 2 && A.L[n - 1].c == 1;
    float *zpart = A.loss_partials + 256;   // [cluster][BM]

    // =================================================================================== forward
    for (int li = 0; li < (fuse_tail ? n - 1 : n); ++li) {
        const SmallStepLayer &L = A.L[li];
        const int r = L.r, c = L.c;
        const int ncl = round4(ceil_div(c, NC));                 // columns per cluster (<= WMAX, checked on the host)
        const int n0 = j * ncl, ncols = min(ncl, c - n0);        // <= 0: nothing for this cluster
        const int kc = round4(ceil_div(r, S));
        const int k0 = q * kc, klen = min(kc, r - k0);           // <= 0: nothing for this rank
        const bool last = li == n - 1;
        float loss_acc = 0.0f;
        const TileMap tm = tile_map(ncl);
        const int ntiles = (ncols > 0 && klen > 0) ? ceil_div(klen, KT) : 0;
        const float *Wl = A.params + L.off_w;
        auto issue_w = [&](int t) {
            const int kb = k0 + t * KT, kn = min(KT, k0 + klen - kb);
            load_tile(bufB + (t & 1) * BUF_B, LDW, Wl + (long long)kb * c + n0, c, kn, ncols, KT, 4 * tm.CG);
        };
        auto issue_a = [&](int t) {
            const int kb = k0 + t * KT, kn = min(KT, k0 + klen - kb);
            load_tile(bufA + (t & 1) * BUF_A, LD, L.act_in + kb, r, B, kn, BM, KT);
            cp_async_commit();
        };
        // the first W tile does not depend on the previous layer: ask for it before waiting for that layer
        if (ntiles > 0) issue_w(0);
        if (li > 0) {
            grid_barrier(bar);
        }
        if (ncols > 0) {
            float acc[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[i][u] = 0.0f;
            auto issue = [&](int t) {
                issue_w(t);
                issue_a(t);
            };
            if (ntiles > 0) issue_a(0);
            for (int t = 0; t < ntiles; ++t) {
                if (t + 1 < ntiles) {
                    issue(t + 1);
                    cp_async_wait<1>();
                } else {
                    cp_async_wait<0>();
                }
                __syncthreads();
                if (tm.active) {
                    const float *as = bufA + (t & 1) * BUF_A, *ws = bufB + (t & 1) * BUF_B;
                    const int seg = KT / tm.KG, kbeg = tm.kg * seg;
#pragma unroll 2
                    for (int k = kbeg; k < kbeg + seg; k += 4) {
                        float4 a[4], w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4 *>(as + (tm.rg + 16 * i) * LD + k);
#pragma unroll
                        for (int u = 0; u < 4; ++u) w[u] = *reinterpret_cast<const float4 *>(ws + (k + u) * LDW + 4 * tm.cg);
                        fma_nn(acc, a, w);
                    }
                }
                __syncthreads();
            }
            // partial sums of this CTA: part[kg][row][col], pitch 4*CG
            const int PLD = 4 * tm.CG;
            if (tm.active) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *reinterpret_cast<float4 *>(part + ((tm.kg * BM) + tm.rg + 16 * i) * PLD + 4 * tm.cg) =
                        make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            }
            fold_and_push(cluster, part, recv, tm.KG, PLD, S, q);
            cluster.sync();
            // this CTA adds the S ranks' tiles of its rows in rank order and finishes the elements
            const float *bias = A.params + L.off_b;
            for (int e = tid; e < RB * ncols; e += T) {
                const int rl = e / ncols, row = q * RB + rl, col = e % ncols;
                if (row >= B) continue;
                const float sum = sum_ranks(recv, S, RB, PLD, rl, col);
                const long long o = (long long)row * c + n0 + col;
                const float z = sum + bias[n0 + col];
                if (!last) {
                    if (L.pre_out) L.pre_out[o] = z;
                    const float a = act_forward(A.act, z);
                    L.act_out[o] = a;
                    // fused tail: this element's term of the output layer's dot product (w_out is a column)
                    if (fuse_tail && li == n - 2) part[rl * PLD + col] = __fmul_rn(a, A.params[A.L[n - 1].off_w + n0 + col]);
                } else if (A.forward_only) {
                    L.act_out[o] = z;
                } else {
                    // MSE and its seed gradient (mlp_train_rust_codegen.rs:793-798)
                    L.act_out[o] = z;
                    const float d = __fsub_rn(z, A.y[o]);
                    loss_acc = __fadd_rn(loss_acc, __fmul_rn(d, d));
                    L.delta[o] = __fdiv_rn(__fmul_rn(2.0f, d), A.nt_global);
                }
            }
            // (no second cluster barrier: the next pushes into `recv` come behind the next grid barrier, or never)
            if (fuse_tail && li == n - 2) {
                // this cluster's partial of every row's output: the terms of the row in column order; cluster 0
                // starts from the output bias (read here, where nobody writes it)
                __syncthreads();
                if (tid < RB && q * RB + tid < B) {
                    float zp = j == 0 ? A.params[A.L[n - 1].off_b] : 0.0f;
                    for (int col = 0; col < ncols; ++col) zp = __fadd_rn(zp, part[tid * PLD + col]);
                    zpart[j * BM + q * RB + tid] = zp;
                }
            }
        }
        if (last && A.forward_only) break;   // inference: the outputs are stored, nothing follows
        if (last) {
            // per-CTA loss partial, fixed tree: warp shuffles, then the 8 warp sums in order
            for (int o = 16; o; o >>= 1) loss_acc += __shfl_xor_sync(0xffffffffu, loss_acc, o);
            if ((tid & 31) == 0) red[tid >> 5] = loss_acc;
            __syncthreads();
            if (tid == 0) {
                float t = 0.0f;
                for (int w = 0; w < T / 32; ++w) t += red[w];
                A.loss_partials[blockIdx.x] = t;
            }
        }
    }

    // =================================================================================== fused tail
    if (fuse_tail) {
        const SmallStepLayer &L = A.L[n - 1];                    // r x 1
        const SmallStepLayer &P = A.L[n - 2];
        const int r = L.r;
        const int kcl = round4(ceil_div(r, NC));
        const int k0 = j * kcl, krows = min(kcl, r - k0);        // rows of w_out this cluster owns; rank q: kk = q, q + S, ..
        const int NAf = ceil_div(P.c, round4(ceil_div(P.c, NC)));   // clusters that wrote a partial
        float *dl = part, *sq = part + BM;                       // seed gradient and squared residual per row
        grid_barrier(bar);
        // (inference: only the outputs are wanted, and only CTA 0 writes them)
        const bool wanted = A.forward_only ? blockIdx.x == 0 : (krows > 0 || blockIdx.x == 0);
        float *zz = bufA;   // [NAf][BM]: all partials, fetched by the whole CTA at once (one L2 latency, not NAf / 8)
        if (wanted) {
#pragma unroll 4
            for (int e = tid; e < NAf * BM; e += T) zz[e] = __ldcg(zpart + e);
        }
        __syncthreads();
        if (tid < BM && wanted) {
            float dv = 0.0f, d2 = 0.0f;
            if (tid < B) {
                float z = zz[tid];
                for (int jj = 1; jj < NAf; ++jj) z = __fadd_rn(z, zz[jj * BM + tid]);
                if (A.forward_only) {
                    L.act_out[tid] = z;
                } else {
                    // MSE and its seed gradient (mlp_train_rust_codegen.rs:793-798)
                    const float d = __fsub_rn(z, A.y[tid]);
                    dv = __fdiv_rn(__fmul_rn(2.0f, d), A.nt_global);
                    d2 = __fmul_rn(d, d);
                    if (blockIdx.x == 0) {
                        L.act_out[tid] = z;
                        L.delta[tid] = dv;
                    }
                }
            }
            dl[tid] = dv;
            sq[tid] = d2;
        }
        __syncthreads();
        if (tid == 0 && !A.forward_only) {
            float t = 0.0f;
            if (blockIdx.x == 0) {
                // the loss is this CTA's alone here: published now, where nobody waits for it
                for (int b = 0; b < B; ++b) t = __fadd_rn(t, sq[b]);
                *A.loss_sum = t;
                if (A.host_loss) *reinterpret_cast<volatile float *>(A.host_loss) = t;
            }
            A.loss_partials[blockIdx.x] = t;
        }
        if (krows > 0 && !A.forward_only) {
            const float wd = OPT == VB200_OPT_ADAMW ? sc.weight_decay : 0.0f;
            // dX of this rank's rows of w_out: delta_prev[b][k] = (delta[b] * w[k]) * f'(saved[b][k])
            const int nk = (krows - q + S - 1) / S;
            for (int e = tid; e < B * nk; e += T) {
                const int b = e / nk, k = k0 + q + S * (e - b * nk);
                const long long o = (long long)b * r + k;
                L.delta_prev[o] = __fmul_rn(__fmul_rn(dl[b], A.params[L.off_w + k]), act_backward(A.act, __ldcg(L.saved_prev + o)));
            }
            __syncthreads();   // every read of the pre-update w_out rows is done
            // dW of the same rows (warp per row; lane l: batch rows l and l + 32, then a fixed shuffle tree), update
            const int lane = tid & 31;
            for (int kk = q + S * (tid >> 5); kk < krows; kk += S * (T / 32)) {
                const int k = k0 + kk;
                const float a0 = lane < B ? __ldcg(L.act_in + (long long)lane * r + k) : 0.0f;
                const float a1 = lane + 32 < B ? __ldcg(L.act_in + (long long)(lane + 32) * r + k) : 0.0f;
                float v = fmaf(a1, dl[lane + 32], __fmul_rn(a0, dl[lane]));
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) {
                    const long long e = L.off_w + k;
                    update_elem<OPT>(A.params + e, A.s1 + e, A.s2 + e, A.grads + e, v, sc, wd);
                }
            }
        }
        if (blockIdx.x == 0 && (tid >> 5) == T / 32 - 1 && !A.forward_only) {
            // the output bias: sum of the seed gradients (nobody reads the bias in this phase)
            const int lane = tid & 31;
            float v = __fadd_rn(dl[lane], dl[lane + 32]);
#pragma unroll
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) {
                const long long e = L.off_b;
                update_elem<OPT>(A.params + e, A.s1 + e, A.s2 + e, A.grads + e, v, sc, 0.0f);
            }
        }
    }

    // =================================================================================== backward
    for (int li = A.forward_only ? -1 : (fuse_tail ? n - 2 : n - 1); li >= 0; --li) {
        const SmallStepLayer &L = A.L[li];
        const int r = L.r, c = L.c;
        const int kcl = round4(ceil_div(r, NC));                 // rows of W per cluster (<= WMAX)
        const int k0 = j * kcl, krows = min(kcl, r - k0);        // <= 0: nothing for this cluster
        const int nc = round4(ceil_div(c, S));
        const int n0 = q * nc, nlen = min(nc, c - n0);           // <= 0: nothing for this rank
        const bool need_dx = li > 0;
        const TileMap tm = tile_map(kcl);                        // for the dX partial [BM x kcl]
        const int ntiles = (krows > 0 && nlen > 0) ? ceil_div(nlen, KT) : 0;
        float *Wl = A.params + L.off_w;
        const int wrows_pad = 4 * tm.CG;                         // rows of the W tile that dX reads (zero beyond krows)
        auto issue_w = [&](int t) {
            const int nb = n0 + t * KT, nn = min(KT, n0 + nlen - nb);
            load_tile(bufB + (t & 1) * BUF_B, LD, Wl + (long long)k0 * c + nb, c, krows, nn, wrows_pad, KT);
        };
        auto issue_d = [&](int t) {
            const int nb = n0 + t * KT, nn = min(KT, n0 + nlen - nb);
            load_tile(bufA + (t & 1) * BUF_A, LD, L.delta + nb, c, B, nn, BM, KT);
            cp_async_commit();
        };
        // W and this layer's input activations were final long ago: ask for them before waiting for the deltas
        if (ntiles > 0) {
            load_tile(actc, LDW, L.act_in + k0, r, B, krows, BM, round4(kcl));
            issue_w(0);
        }
        grid_barrier(bar);
        if (li == 0 && blockIdx.x == 0 && tid == 0 && A.host_status) {
            // the step's last barrier: CTA 0 passed every one, so no CTA can still be about to give up on one and
            // the status word is final; published here, where nobody waits for it
            *reinterpret_cast<volatile unsigned *>(A.host_status) = *reinterpret_cast<volatile unsigned *>(A.status);
        }
        if (krows > 0) {
            float acc[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[i][u] = 0.0f;
            auto issue = [&](int t) {
                issue_w(t);
                issue_d(t);
            };
            if (ntiles > 0) issue_d(0);
            for (int t = 0; t < ntiles; ++t) {
                if (t + 1 < ntiles) {
                    issue(t + 1);
                    cp_async_wait<1>();
                } else {
                    cp_async_wait<0>();
                }
                __syncthreads();
                const float *ds = bufA + (t & 1) * BUF_A, *ws = bufB + (t & 1) * BUF_B;
                const int nb = n0 + t * KT, nn = min(KT, n0 + nlen - nb);
                // ---- bias gradient: of the NA clusters that own rows of this W, cluster j takes the tile's columns
                // j, j + NA, ... (all of them hold the same delta tile).  The sums are taken by warp 0 inside its first
                // block of products (lane l: columns 4l .. 4l+3, rows ascending); the parameter and its state are asked
                // for behind it and used at the end of the tile.
                float db_g = 0.0f, db_p = 0.0f, db_s1 = 0.0f, db_s2 = 0.0f;
                long long db_e = -1;
                auto db_finish = [&]() {
                    update_one<OPT>(db_p, db_s1, db_s2, db_g, sc, 0.0f);
                    A.params[db_e] = db_p;
                    if (OPT != VB200_OPT_SGD) A.s1[db_e] = db_s1;
                    if (OPT == VB200_OPT_ADAM || OPT == VB200_OPT_ADAMW) A.s2[db_e] = db_s2;
                    A.grads[db_e] = db_g;
                };
                // ---- dW block = act^T . delta (sum over the batch, ascending), then the optimizer on it.  A thread
                // owns 4 columns and RPT rows of the block; RPT shrinks with the slab so that all eight warps have rows.
                auto dw_block = [&](auto rpt_tag) {
                    constexpr int RPT = decltype(rpt_tag)::value;
                    const int ng = tid & 31, kgp = tid >> 5;     // columns 4*ng .., rows kgp*RPT + 8*RPT*pass ..
                    for (int pass = 0; pass * 8 * RPT < kcl; ++pass) {
                        const int kk0 = kgp * RPT + 8 * RPT * pass;
                        if (kk0 >= kcl) break;
                        float g[RPT][4];
#pragma unroll
                        for (int i = 0; i < RPT; ++i)
#pragma unroll
                            for (int u = 0; u < 4; ++u) g[i][u] = 0.0f;
                        // optimizer state of the rows, asked for before the products so that its latency
                        // hides behind them (the weights themselves sit in the shared-memory tile)
                        constexpr bool HAS1 = (OPT != VB200_OPT_SGD);
                        constexpr bool HAS2 = (OPT == VB200_OPT_ADAM || OPT == VB200_OPT_ADAMW);
                        const bool vec = (c & 3) == 0 && 4 * ng + 3 < nn;   // offsets and n0, nb are multiples of 4
                        float4 st1[RPT], st2[RPT];
#pragma unroll
                        for (int i = 0; i < RPT; ++i) {
                            st1[i] = st2[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                            if (vec && kk0 + i < krows) {
                                const long long e = L.off_w + (long long)(k0 + kk0 + i) * c + nb + 4 * ng;
                                if (HAS1) st1[i] = load_early(A.s1 + e);
                                if (HAS2) st2[i] = load_early(A.s2 + e);
                            }
                        }
                        const bool do_db = kgp == 0 && pass == 0;
                        float cs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
                        for (int b = 0; b < B; ++b) {
                            float a4[RPT];
                            if (RPT == 4) {
                                const float4 av = *reinterpret_cast<const float4 *>(actc + b * LDW + kk0);
                                a4[0] = av.x; a4[RPT > 1 ? 1 : 0] = av.y; a4[RPT > 2 ? 2 : 0] = av.z; a4[RPT > 3 ? 3 : 0] = av.w;
                            } else if (RPT == 2) {
                                const float2 av = *reinterpret_cast<const float2 *>(actc + b * LDW + kk0);
                                a4[0] = av.x; a4[RPT > 1 ? 1 : 0] = av.y;
                            } else {
                                a4[0] = actc[b * LDW + kk0];
                            }
                            const float4 dv = *reinterpret_cast<const float4 *>(ds + b * LD + 4 * ng);
#pragma unroll
                            for (int i = 0; i < RPT; ++i) {
                                g[i][0] = fmaf(a4[i], dv.x, g[i][0]);
                                g[i][1] = fmaf(a4[i], dv.y, g[i][1]);
                                g[i][2] = fmaf(a4[i], dv.z, g[i][2]);
                                g[i][3] = fmaf(a4[i], dv.w, g[i][3]);
                            }
                            if (do_db) {   // warp 0: the column sums of the delta tile ride along (rows ascending)
                                cs[0] += dv.x; cs[1] += dv.y; cs[2] += dv.z; cs[3] += dv.w;
                            }
                        }
                        if (do_db) {
                            const int NA = ceil_div(r, kcl);   // clusters with krows > 0
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const int col = 4 * ng + u;
                                if (col < nn && col % NA == j) {
                                    if (db_e >= 0) db_finish();   // NA < 4: more than one column for this lane
                                    db_g = cs[u];
                                    db_e = L.off_b + nb + col;
                                    db_p = A.params[db_e];
                                    if (OPT != VB200_OPT_SGD) db_s1 = __ldcs(A.s1 + db_e);
                                    if (OPT == VB200_OPT_ADAM || OPT == VB200_OPT_ADAMW) db_s2 = __ldcs(A.s2 + db_e);
                                }
                            }
                        }
                        const float wd = OPT == VB200_OPT_ADAMW ? sc.weight_decay : 0.0f;
                        if (c == 1) {
                            // a width-one layer's W is a column: this thread's rows are consecutive floats, updated
                            // as one group of four where all four exist (k0 and kk0 are then multiples of 4)
                            if (ng == 0 && kk0 < krows) {
                                const long long e = L.off_w + k0 + kk0;
                                if (RPT == 4 && kk0 + 3 < krows) {
                                    float4 pv = *reinterpret_cast<const float4 *>(A.params + e);
                                    float4 a1 = HAS1 ? __ldcs(reinterpret_cast<const float4 *>(A.s1 + e)) : make_float4(0, 0, 0, 0);
                                    float4 a2 = HAS2 ? __ldcs(reinterpret_cast<const float4 *>(A.s2 + e)) : make_float4(0, 0, 0, 0);
                                    update_one<OPT>(pv.x, a1.x, a2.x, g[0][0], sc, wd);
                                    update_one<OPT>(pv.y, a1.y, a2.y, g[RPT > 1 ? 1 : 0][0], sc, wd);
                                    update_one<OPT>(pv.z, a1.z, a2.z, g[RPT > 2 ? 2 : 0][0], sc, wd);
                                    update_one<OPT>(pv.w, a1.w, a2.w, g[RPT > 3 ? 3 : 0][0], sc, wd);
                                    *reinterpret_cast<float4 *>(A.params + e) = pv;
                                    if (HAS1) *reinterpret_cast<float4 *>(A.s1 + e) = a1;
                                    if (HAS2) *reinterpret_cast<float4 *>(A.s2 + e) = a2;
                                    *reinterpret_cast<float4 *>(A.grads + e) =
                                        make_float4(g[0][0], g[RPT > 1 ? 1 : 0][0], g[RPT > 2 ? 2 : 0][0], g[RPT > 3 ? 3 : 0][0]);
                                } else {
#pragma unroll
                                    for (int i = 0; i < RPT; ++i)
                                        if (kk0 + i < krows)
                                            update_elem<OPT>(A.params + e + i, A.s1 + e + i, A.s2 + e + i, A.grads + e + i, g[i][0], sc, wd);
                                }
                            }
                            continue;
                        }
                        if (vec) {
                            // all rows of the thread side by side (the optimizer's chains interleave), then the stores
                            float4 pv[RPT];
#pragma unroll
                            for (int i = 0; i < RPT; ++i)   // pre-update W from the tile (zero rows beyond krows)
                                pv[i] = *reinterpret_cast<const float4 *>(ws + (kk0 + i) * LD + 4 * ng);
                            update_rows<OPT, RPT>(pv, st1, st2, g, sc, wd);
#pragma unroll
                            for (int i = 0; i < RPT; ++i) {
                                if (kk0 + i >= krows) continue;
                                const long long e = L.off_w + (long long)(k0 + kk0 + i) * c + nb + 4 * ng;
                                *reinterpret_cast<float4 *>(A.params + e) = pv[i];
                                if (HAS1) *reinterpret_cast<float4 *>(A.s1 + e) = st1[i];
                                if (HAS2) *reinterpret_cast<float4 *>(A.s2 + e) = st2[i];
                                *reinterpret_cast<float4 *>(A.grads + e) = make_float4(g[i][0], g[i][1], g[i][2], g[i][3]);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < RPT; ++i) {
                                const int kk = kk0 + i;
                                if (kk >= krows) continue;
                                const long long e = L.off_w + (long long)(k0 + kk) * c + nb + 4 * ng;
#pragma unroll
                                for (int u = 0; u < 4; ++u)
                                    if (4 * ng + u < nn)
                                        update_elem<OPT>(A.params + e + u, A.s1 + e + u, A.s2 + e + u, A.grads + e + u, g[i][u], sc, wd);
                            }
                        }
                    }
                };
                dw_block(std::integral_constant<int, 2>{});
                // ---- partial of dX = delta . W^T over this tile's columns, from the pre-update W in shared memory
                if (need_dx && tm.active) {
                    const int seg = KT / tm.KG, nbeg = tm.kg * seg;
#pragma unroll 2
                    for (int nn4 = nbeg; nn4 < nbeg + seg; nn4 += 4) {
                        float4 d[4], w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) d[i] = *reinterpret_cast<const float4 *>(ds + (tm.rg + 16 * i) * LD + nn4);
#pragma unroll
                        for (int u = 0; u < 4; ++u) w[u] = *reinterpret_cast<const float4 *>(ws + (tm.cg + tm.CG * u) * LD + nn4);
                        fma_nt(acc, d, w);
                    }
                }
                if (db_e >= 0) db_finish();
                __syncthreads();
            }
            if (need_dx) {
                // partials: part[kg][row][kk], kk = cg + CG*u, pitch 4*CG
                const int PLD = 4 * tm.CG;
                if (tm.active) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int u = 0; u < 4; ++u) part[((tm.kg * BM) + tm.rg + 16 * i) * PLD + tm.cg + tm.CG * u] = acc[i][u];
                }
                fold_and_push(cluster, part, recv, tm.KG, PLD, S, q);
                cluster.sync();
                for (int e = tid; e < RB * krows; e += T) {
                    const int rl = e / krows, row = q * RB + rl, kk = e % krows;
                    if (row >= B) continue;
                    const float sum = sum_ranks(recv, S, RB, PLD, rl, kk);
                    const long long o = (long long)row * r + k0 + kk;
                    L.delta_prev[o] = sum * act_backward(A.act, __ldcg(L.saved_prev + o));
                }
                // (no second cluster barrier: the next phase's pushes come behind its grid barrier)
            }
        }
    }
    if (blockIdx.x == 0 && !A.forward_only && !fuse_tail) {
        // The loss: every CTA's partial (final since the barrier behind the last forward layer), added in CTA
        // order.  Done here, where nobody waits for CTA 0: warp 0 fetches the partials in parallel, thread 0 adds.
        float *lp = bufA;   // the staging buffers are idle by now
        for (unsigned b = tid; b < gridDim.x; b += T) lp[b] = __ldcg(A.loss_partials + b);
        __syncthreads();
        if (tid == 0) {
            float t = 0.0f;
            for (unsigned b = 0; b < gridDim.x; ++b) t += lp[b];
            *A.loss_sum = t;
            if (A.host_loss) *reinterpret_cast<volatile float *>(A.host_loss) = t;
        }
    }
    cluster.sync();   // no CTA leaves while a peer may still write into its shared memory
}

bool g_smem_set[kMaxDevices][5] = {};

template <int OPT>
cudaError_t launch_opt(const SmallStepArgs &args, int grid, int S, cudaStream_t s) {
    const int dev = current_device();
    const size_t smem = SMEM_FLOATS * sizeof(float);
    if (!g_smem_set[dev][OPT]) {
        cudaError_t e = cudaFuncSetAttribute(small_step_kernel<OPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        g_smem_set[dev][OPT] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(T);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)S;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeCooperative;   // all CTAs resident at once: they wait on one another
    at[1].val.cooperative = 1;
    cfg.attrs = at;
    // VOLTA_B200_STEP_COOP=0 drops the cooperative attribute (the grid is sized to be resident either way)
    static const bool coop = [] { const char *e = getenv("VOLTA_B200_STEP_COOP"); return !(e && e[0] == '0'); }();
    cfg.numAttrs = coop ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, small_step_kernel<OPT>, args);
}

template <int OPT>
int max_clusters(int S) {
    const size_t smem = SMEM_FLOATS * sizeof(float);
    if (cudaFuncSetAttribute(small_step_kernel<OPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)S);
    cfg.blockDim = dim3(T);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)S;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, small_step_kernel<OPT>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

}  // namespace

// Shape limits of the persistent step (a function of the topology and of the cluster count alone).
bool small_step_shape_ok(const int *layers, int n_sizes, int batch, int clusters) {
    if (batch < 1 || batch > BM || n_sizes < 2 || n_sizes - 1 > kSmallStepMaxLayers || clusters < 1) return false;
    for (int i = 0; i < n_sizes; ++i)
        if (((layers[i] + clusters - 1) / clusters + 3) / 4 * 4 > WMAX) return false;
    return true;
}

// Grid of the persistent step on the current device: `*cluster` CTAs per cluster (4 unless
// VOLTA_B200_STEP_CLUSTER says 1, 2 or 8) times as many clusters as are resident at once, at most one
// CTA per SM.  Returns 0 when the device cannot hold it.
int small_step_grid(int optimizer, int *cluster) {
    static const int want = [] { const char *e = getenv("VOLTA_B200_STEP_CLUSTER"); int v = e ? atoi(e) : 4; return (v == 1 || v == 2 || v == 4 || v == 8) ? v : 4; }();
    int n = 0;
    switch (optimizer) {
    case VB200_OPT_SGD: n = max_clusters<VB200_OPT_SGD>(want); break;
    case VB200_OPT_ADAM: n = max_clusters<VB200_OPT_ADAM>(want); break;
    case VB200_OPT_ADAMW: n = max_clusters<VB200_OPT_ADAMW>(want); break;
    case VB200_OPT_ADAGRAD: n = max_clusters<VB200_OPT_ADAGRAD>(want); break;
    case VB200_OPT_SGD_MOMENTUM: n = max_clusters<VB200_OPT_SGD_MOMENTUM>(want); break;
    }
    const int by_sm = device_sm_count() / want;
    if (n > by_sm) n = by_sm;
    *cluster = want;
    return n > 0 ? n * want : 0;
}

cudaError_t launch_small_step(const SmallStepArgs &args, int grid, int cluster, cudaStream_t s) {
    switch (args.opt) {
    case VB200_OPT_SGD: return launch_opt<VB200_OPT_SGD>(args, grid, cluster, s);
    case VB200_OPT_ADAM: return launch_opt<VB200_OPT_ADAM>(args, grid, cluster, s);
    case VB200_OPT_ADAMW: return launch_opt<VB200_OPT_ADAMW>(args, grid, cluster, s);
    case VB200_OPT_ADAGRAD: return launch_opt<VB200_OPT_ADAGRAD>(args, grid, cluster, s);
    case VB200_OPT_SGD_MOMENTUM: return launch_opt<VB200_OPT_SGD_MOMENTUM>(args, grid, cluster, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace vb
