// Data-parallel gradient exchange fused with the optimizer, over peer memory (NVLink P2P).
//
// The NCCL path all-reduces every gradient bucket and then every rank runs the same optimizer over
// all parameters.  Here the collective and the update are ONE kernel per bucket: rank r owns the
// r-th share of the bucket; it reads that share of every rank's gradient buffer with plain 128-bit
// peer loads, adds them in rank order 0..N-1 (so the sum is the same bits on every run), applies the
// optimizer to its share (only the owner keeps optimizer state for it), and stores the new
// parameters into every rank's arena (reduce-scatter + update + all-gather).  Optimizer traffic per
// GPU drops by the rank count; gradients cross NVLink once and parameters once.
//
// Ordering between ranks uses flag words in each arena: before a bucket's kernel every rank announces
// "my backward for this layer is done" and waits for all others (so nobody's weights are overwritten
// while it still reads them, and every gradient is final); one more barrier at the end of the step
// makes all updates visible before the next forward.  Waits are bounded (4 s unless the handle's
// configuration says otherwise): on expiry a status bit is set, and from then on every barrier and
// every reduce-update kernel of the handle returns at once without reading or writing any rank's
// memory - a missing rank neither hangs the GPU nor gets a partial sum applied, and the host
// refuses further steps with VB200_ERR_DEVICE_WAIT.
//
// Exchange by copy (dp_gather_update_kernel, the handle's dp_exchange = VB200_DP_PEER_COPY): the same flag
// barriers, but the gradients travel by the copy engines - the host side enqueues, per layer bucket, one
// device-to-device copy of the bucket into this rank's receive slot in every peer's arena as soon as dW exists,
// so that no SM is taken from the backward GEMMs that run meanwhile (a collective kernel that holds an SM for
// the length of its transfer also blocks that SM's partner for the CTA-pair GEMM).  After the bucket's
// barrier every rank holds all N copies locally; one streaming kernel adds them in rank order 0..N-1, stores
// the sum as the gradient and applies the optimizer to the whole bucket: every rank keeps full optimizer
// state and identical parameters without a second transfer.  N-1 times the gradient bytes cross NVLink per
// rank instead of 2(N-1)/N, all of it underneath the backward pass.
// The reference has no collective of any kind; parity target is the full-batch CPU oracle.
#include "vb_common.cuh"
#include "vb_optimizer.cuh"

namespace vb {
namespace {

constexpr unsigned ST_DP_BARRIER = kStatusDpBarrier;

__device__ __forceinline__ unsigned long long dp_global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void dp_barrier_kernel(PeerTable peers, long long flags_off, int world, int rank,
                                  const StepScalars *__restrict__ scalars, unsigned stride, unsigned index,
                                  unsigned int *status, unsigned long long wait_ns) {
    pdl_wait();
    const int t = threadIdx.x;
    if (t >= world) return;
    // an earlier barrier of this handle gave up: some rank is missing, leave every peer alone
    if (*reinterpret_cast<volatile unsigned int *>(status) & ST_DP_BARRIER) return;
    const unsigned value = scalars->epoch * stride + index;
    __threadfence_system();   // everything this GPU wrote before the barrier is visible to its peers
    volatile unsigned *theirs = reinterpret_cast<volatile unsigned *>(peers.base[t] + flags_off) + rank;
    *theirs = value;
    volatile unsigned *mine = reinterpret_cast<volatile unsigned *>(peers.base[rank] + flags_off) + t;
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
        if ((int)(*mine - value) >= 0) break;
        if ((it & 1023u) == 1023u) {
            unsigned long long now = dp_global_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > wait_ns) {
                atomicOr(status, ST_DP_BARRIER);
                break;
            }
        }
    }
    __threadfence_system();
}

template <int OPT>
__global__ void __launch_bounds__(256) dp_reduce_update_kernel(PeerTable peers, long long params_off, long long grads_off,
                                                               long long s1_off, long long s2_off, long long seg_begin,
                                                               long long seg_len, long long n_decay, int world, int rank,
                                                               const StepScalars *__restrict__ scp, long long loss_off,
                                                               const unsigned int *__restrict__ status) {
    pdl_wait();
    // the barrier before this kernel gave up: gradients are partial or stale and a peer's arena may be
    // gone, so nothing is read from or written to any rank and the parameters stay as they were
    if (*reinterpret_cast<const volatile unsigned int *>(status) & ST_DP_BARRIER) return;
    const StepScalars sc = *scp;
    constexpr bool HAS1 = (OPT != VB200_OPT_SGD);
    constexpr bool HAS2 = (OPT == VB200_OPT_ADAM || OPT == VB200_OPT_ADAMW);
    // this rank's share of the segment, in float4 units (segments are multiples of 64 floats)
    const long long seg4 = seg_len >> 2;
    const long long per = (seg4 + world - 1) / world;
    const long long lo = rank * per, hi = (lo + per < seg4) ? (lo + per) : seg4;
    float4 *my_p = reinterpret_cast<float4 *>(peers.base[rank] + params_off) + (seg_begin >> 2);
    float4 *my_s1 = reinterpret_cast<float4 *>(peers.base[rank] + s1_off) + (seg_begin >> 2);
    float4 *my_s2 = reinterpret_cast<float4 *>(peers.base[rank] + s2_off) + (seg_begin >> 2);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += stride) {
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < world; ++q) {   // fixed rank order
            const float4 v = __ldcv(reinterpret_cast<const float4 *>(peers.base[q] + grads_off) + (seg_begin >> 2) + i);
            g.x += v.x; g.y += v.y; g.z += v.z; g.w += v.w;
        }
        float4 pv = my_p[i];
        float4 a = HAS1 ? my_s1[i] : make_float4(0, 0, 0, 0);
        float4 b = HAS2 ? my_s2[i] : make_float4(0, 0, 0, 0);
        const long long e = seg_begin + (i << 2);
        const float wd0 = (OPT == VB200_OPT_ADAMW && e + 0 < n_decay) ? sc.weight_decay : 0.0f;
        const float wd1 = (OPT == VB200_OPT_ADAMW && e + 1 < n_decay) ? sc.weight_decay : 0.0f;
        const float wd2 = (OPT == VB200_OPT_ADAMW && e + 2 < n_decay) ? sc.weight_decay : 0.0f;
        const float wd3 = (OPT == VB200_OPT_ADAMW && e + 3 < n_decay) ? sc.weight_decay : 0.0f;
        update_one<OPT>(pv.x, a.x, b.x, g.x, sc, wd0);
        update_one<OPT>(pv.y, a.y, b.y, g.y, sc, wd1);
        update_one<OPT>(pv.z, a.z, b.z, g.z, sc, wd2);
        update_one<OPT>(pv.w, a.w, b.w, g.w, sc, wd3);
        if (HAS1) my_s1[i] = a;
        if (HAS2) my_s2[i] = b;
        for (int q = 0; q < world; ++q)   // all-gather: the new parameters land in every rank's arena
            reinterpret_cast<float4 *>(peers.base[q] + params_off)[(seg_begin >> 2) + i] = pv;
    }
    // the loss travels with the last bucket: every rank adds all ranks' partial sums in rank order
    if (loss_off >= 0 && blockIdx.x == 0 && threadIdx.x == 0) {
        float total = 0.0f;
        for (int q = 0; q < world; ++q) total += *reinterpret_cast<volatile const float *>(peers.base[q] + loss_off);
        reinterpret_cast<float *>(peers.base[rank] + loss_off)[1] = total;
    }
    __threadfence_system();
}

// The copy exchange's consumer: every rank's copy of the segment is local by now (own gradients in `grads`,
// rank q's in its receive slot), so this is the streaming optimizer with `world` gradient operands.
template <int OPT>
__global__ void __launch_bounds__(256) dp_gather_update_kernel(float *__restrict__ params, float *__restrict__ s1p,
                                                               float *__restrict__ s2p, float *__restrict__ grads,
                                                               const float *__restrict__ recv, long long slot_floats,
                                                               long long seg_begin, long long seg_len, long long n_decay,
                                                               int world, int rank, const StepScalars *__restrict__ scp,
                                                               long long loss_index, const unsigned int *__restrict__ status) {
    pdl_wait();
    if (*reinterpret_cast<const volatile unsigned int *>(status) & ST_DP_BARRIER) return;
    const StepScalars sc = *scp;
    constexpr bool HAS1 = (OPT != VB200_OPT_SGD);
    constexpr bool HAS2 = (OPT == VB200_OPT_ADAM || OPT == VB200_OPT_ADAMW);
    const long long seg4 = seg_len >> 2, b4 = seg_begin >> 2;
    float4 *g4 = reinterpret_cast<float4 *>(grads) + b4;
    float4 *p4 = reinterpret_cast<float4 *>(params) + b4;
    float4 *a4 = reinterpret_cast<float4 *>(s1p) + b4;
    float4 *c4 = reinterpret_cast<float4 *>(s2p) + b4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < seg4; i += stride) {
        float4 v[kMaxPeers];
#pragma unroll
        for (int q = 0; q < kMaxPeers; ++q)   // all loads first, then the sum in rank order
            if (q < world)
                v[q] = q == rank ? g4[i] : __ldcs(reinterpret_cast<const float4 *>(recv + q * slot_floats) + b4 + i);
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int q = 0; q < kMaxPeers; ++q)
            if (q < world) { g.x += v[q].x; g.y += v[q].y; g.z += v[q].z; g.w += v[q].w; }
        float4 pv = p4[i];
        float4 a = HAS1 ? a4[i] : make_float4(0, 0, 0, 0);
        float4 b = HAS2 ? c4[i] : make_float4(0, 0, 0, 0);
        const long long e = seg_begin + (i << 2);
        const float wd0 = (OPT == VB200_OPT_ADAMW && e + 0 < n_decay) ? sc.weight_decay : 0.0f;
        const float wd1 = (OPT == VB200_OPT_ADAMW && e + 1 < n_decay) ? sc.weight_decay : 0.0f;
        const float wd2 = (OPT == VB200_OPT_ADAMW && e + 2 < n_decay) ? sc.weight_decay : 0.0f;
        const float wd3 = (OPT == VB200_OPT_ADAMW && e + 3 < n_decay) ? sc.weight_decay : 0.0f;
        update_one<OPT>(pv.x, a.x, b.x, g.x, sc, wd0);
        update_one<OPT>(pv.y, a.y, b.y, g.y, sc, wd1);
        update_one<OPT>(pv.z, a.z, b.z, g.z, sc, wd2);
        update_one<OPT>(pv.w, a.w, b.w, g.w, sc, wd3);
        p4[i] = pv;
        if (HAS1) a4[i] = a;
        if (HAS2) c4[i] = b;
        g4[i] = g;   // the global gradient, as the all-reduce path leaves it
    }
    if (loss_index >= 0 && blockIdx.x == 0 && threadIdx.x == 0) {
        float total = 0.0f;
        for (int q = 0; q < world; ++q) total += q == rank ? grads[loss_index] : recv[q * slot_floats + loss_index];
        grads[loss_index + 1] = total;
    }
}

}  // namespace

cudaError_t launch_dp_gather_update(int optimizer, float *params, float *s1, float *s2, float *grads, const float *recv,
                                    long long slot_floats, long long seg_begin, long long seg_len, long long n_decay,
                                    int world, int rank, const StepScalars *scalars, long long loss_index,
                                    const unsigned int *status, cudaStream_t s) {
    if (seg_len <= 0 || (seg_len & 3) || (seg_begin & 3) || (slot_floats & 3) || world < 1 || world > kMaxPeers)
        return cudaErrorInvalidValue;
    long long want = ((seg_len >> 2) + 255) / 256;
    const int cap = device_sm_count() * 8;
    int blocks = (int)(want < 1 ? 1 : (want > cap ? cap : want));
#define VB_DP_LAUNCH(O)                                                                                              \
    return launch_pdl(dp_gather_update_kernel<O>, dim3(blocks), dim3(256), 0, s, params, s1, s2, grads, recv, slot_floats, \
                      seg_begin, seg_len, n_decay, world, rank, scalars, loss_index, status)
    switch (optimizer) {
    case VB200_OPT_SGD: VB_DP_LAUNCH(VB200_OPT_SGD);
    case VB200_OPT_ADAM: VB_DP_LAUNCH(VB200_OPT_ADAM);
    case VB200_OPT_ADAMW: VB_DP_LAUNCH(VB200_OPT_ADAMW);
    case VB200_OPT_ADAGRAD: VB_DP_LAUNCH(VB200_OPT_ADAGRAD);
    case VB200_OPT_SGD_MOMENTUM: VB_DP_LAUNCH(VB200_OPT_SGD_MOMENTUM);
    }
#undef VB_DP_LAUNCH
    return cudaErrorInvalidValue;
}

cudaError_t launch_dp_barrier(const PeerTable &peers, long long flags_off, int world, int rank,
                              const StepScalars *scalars, unsigned stride, unsigned index, unsigned int *status,
                              unsigned long long wait_ns, cudaStream_t s) {
    return launch_pdl(dp_barrier_kernel, dim3(1), dim3(32), 0, s, peers, flags_off, world, rank, scalars, stride, index, status,
                      wait_ns);
}

cudaError_t launch_dp_reduce_update(int optimizer, const PeerTable &peers, long long params_off, long long grads_off,
                                    long long s1_off, long long s2_off, long long seg_begin, long long seg_len,
                                    long long n_decay, int world, int rank, const StepScalars *scalars,
                                    long long loss_off, const unsigned int *status, cudaStream_t s) {
    if (seg_len <= 0 || (seg_len & 3) || (seg_begin & 3)) return cudaErrorInvalidValue;
    const long long per = ((seg_len >> 2) + world - 1) / world;
    long long want = (per + 255) / 256;
    int blocks = (int)(want < 1 ? 1 : (want > 148 * 4 ? 148 * 4 : want));
#define VB_DP_LAUNCH(O)                                                                                              \
    return launch_pdl(dp_reduce_update_kernel<O>, dim3(blocks), dim3(256), 0, s, peers, params_off, grads_off, s1_off, \
                      s2_off, seg_begin, seg_len, n_decay, world, rank, scalars, loss_off, status)
    switch (optimizer) {
    case VB200_OPT_SGD: VB_DP_LAUNCH(VB200_OPT_SGD);
    case VB200_OPT_ADAM: VB_DP_LAUNCH(VB200_OPT_ADAM);
    case VB200_OPT_ADAMW: VB_DP_LAUNCH(VB200_OPT_ADAMW);
    case VB200_OPT_ADAGRAD: VB_DP_LAUNCH(VB200_OPT_ADAGRAD);
    case VB200_OPT_SGD_MOMENTUM: VB_DP_LAUNCH(VB200_OPT_SGD_MOMENTUM);
    }
#undef VB_DP_LAUNCH
    return cudaErrorInvalidValue;
}

}  // namespace vb
