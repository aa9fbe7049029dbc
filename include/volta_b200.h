/*
 * libvolta_b200 — C ABI of the B200 (sm_100a) implementation of Volta's compiled MLP
 * training step.  Plain pointers and sizes only; no C++ or torch types cross this line.
 *
 * Two groups of entry points:
 *
 *  1. volta_b200_*  — exported by libvolta_b200.so.  A handle-based, topology-agnostic
 *     restatement of the six functions every Volta training library exports, plus the
 *     few extensions the GPU build needs (topology passed at run time instead of being
 *     compiled in, device-resident inputs, data-parallel ranks, error reporting).
 *
 *  2. volta_train_* — the reference's own symbol names.  They are exported by the small
 *     per-model library that `volta-b200-codegen` emits (include/volta_train.h), whose
 *     bodies forward to group 1 with the model's topology compiled in, exactly as the
 *     reference compiles one shared object per model.
 *
 * Every function cites the reference interface it replaces, as
 * src/engine/ir/codegen/mlp_train_rust_codegen.rs:<lines> in the Volta source tree.
 */
#ifndef VOLTA_B200_H
#define VOLTA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VB200_MAX_LAYERS 32

/* Hidden-layer activation (MlpTopology::activation, mlp_train_rust_codegen.rs:268-275).
 * SOFTMAX is the row-wise softmax over each hidden layer's outputs (:727-740, backward :898-906). */
enum { VB200_ACT_RELU = 0, VB200_ACT_SIGMOID = 1, VB200_ACT_TANH = 2, VB200_ACT_LEAKY_RELU = 3,
       VB200_ACT_SILU = 4, VB200_ACT_GELU = 5, VB200_ACT_SOFTMAX = 6 };

/* Optimizer (MlpTopology::optimizer, mlp_train_rust_codegen.rs:263-267).  SGD with
 * momentum has no counterpart in the reference; it is an extension. */
enum { VB200_OPT_SGD = 0, VB200_OPT_ADAM = 1, VB200_OPT_ADAMW = 2, VB200_OPT_ADAGRAD = 3,
       VB200_OPT_SGD_MOMENTUM = 4 };

/* GEMM path selection. AUTO routes each GEMM by shape: the tcgen05 kernels for large ones (CTA pairs
 * with cta_group::2 on 256 x 256 tiles, or single CTAs on 128 x 128 tiles, either with K split over
 * concurrent CTAs where that fills the GPU better), FFMA with split-K for small ones, and for forward
 * GEMMs of at most 8 rows - single-sample inference - a kernel whose CTA clusters split the input
 * features and reduce through distributed shared memory.  FFMA and TENSOR force one family for every
 * GEMM that can take it; TENSOR_PAIR forces the CTA-pair kernel for outputs of at least 256 x 256
 * (other shapes go as under TENSOR). */
enum { VB200_GEMM_AUTO = 0, VB200_GEMM_FFMA = 1, VB200_GEMM_TENSOR = 2, VB200_GEMM_TENSOR_PAIR = 3 };
/* how data-parallel ranks exchange gradients once volta_b200_dp_attach_peers has been called (before that,
 * and always with VB200_DP_NCCL, gradient buckets are all-reduced by NCCL) */
enum { VB200_DP_NCCL = 0, VB200_DP_PEER_KERNEL = 1, VB200_DP_PEER_COPY = 2 };

/* Error codes (0 = success). The reference reports no errors on this path
 * (void functions, mlp_train_rust_codegen.rs:670-699); the replacement never traps and
 * reports through these codes and volta_b200_last_error(). */
enum { VB200_OK = 0, VB200_ERR_INVALID = 1, VB200_ERR_CUDA = 2, VB200_ERR_OOM = 3, VB200_ERR_NCCL = 4,
       VB200_ERR_DEVICE_WAIT = 5, VB200_ERR_UNSUPPORTED = 6, VB200_ERR_TOO_LARGE = 7, VB200_ERR_NONFINITE = 8 };

/* Replaces MlpTopology (mlp_train_rust_codegen.rs:28-39) plus the `batch` argument of
 * volta_train_init.  Hyper-parameters other than lr are fixed in the reference's
 * template (beta1 0.9, beta2 0.999, eps 1e-8, AdamW decay 0.01 on weights only,
 * leaky slope 0.01: mlp_train_rust_codegen.rs:573, 807-813); a zero here selects
 * those defaults. */
typedef struct vb200_config {
    int32_t n_sizes;                   /* number of layer widths (>= 2) */
    int32_t layers[VB200_MAX_LAYERS];  /* widths L0..Ln */
    int32_t activation;                /* VB200_ACT_* */
    int32_t optimizer;                 /* VB200_OPT_* */
    int32_t batch;                     /* rows this handle processes per step (its shard) */
    int32_t global_batch;              /* rows over all ranks; 0 = batch */
    int32_t world_size;                /* data-parallel ranks; 0 or 1 = single GPU */
    int32_t rank;
    uint8_t nccl_unique_id[128];       /* from volta_b200_dp_unique_id, same on all ranks */
    float momentum;                    /* SGD momentum; 0 = 0.9 */
    float weight_decay;                /* AdamW; 0 = 0.01 */
    int32_t gemm_path;                 /* VB200_GEMM_* */
    int32_t use_graph;                 /* 0 = default (captured CUDA graph), 1 = graph, 2 = plain launches */
    int32_t force_dp;                  /* 1: build the data-parallel path (communicator, bucketed all-reduce)
                                          even for world_size 1, so it can be exercised on one GPU */
    int32_t fuse_sgd;                  /* 1: plain SGD on one GPU folds the update into the dW GEMM epilogue (the
                                          reference's sgd_fused_tn); gradients of those layers are then never
                                          materialised and volta_b200_get_grads does not return them */
    /* MlpTopology's remaining switches (mlp_train_rust_codegen.rs:34-38), all off when zero.  Every hidden
     * layer's output goes through activation -> LayerNorm -> dropout, in that order (:725-788). */
    int32_t use_layernorm;             /* 1: LayerNorm over each hidden row (biased variance, eps 1e-5, gamma 1 /
                                          beta 0 at start), whose gamma/beta take a plain SGD step with the
                                          step's lr whatever the optimizer is (:744-772, 829-887) */
    float dropout_p;                   /* in (0,1): inverted dropout; the keep mask is the reference's LCG stream
                                          (seed 12345678, one draw per hidden element in layer, row, column order,
                                          keep when (state >> 33) / 2^31 >= p; :773-788).  Data-parallel ranks
                                          draw the slice of that stream that belongs to their rows */
    float clip_grad;                   /* > 0: the template's "clip": when the norm over ALL deltas exceeds this,
                                          the deltas are scaled by clip/norm after the bias gradients were taken,
                                          so dW shrinks and db does not (:936-955) */
    int32_t device_wait_ms;            /* how long a data-parallel barrier waits for the other ranks before it gives
                                          up (the step then applies no update and the handle reports
                                          VB200_ERR_DEVICE_WAIT); 0 = $VOLTA_B200_WAIT_MS, else 4000 */
    int32_t check_finite;              /* 1: after every step one more kernel looks for inf/NaN in the loss, the
                                          gradients, the parameters and the optimizer state, as the reference's
                                          runtime loop does (src/engine/ir/train.rs:670-773; its generated step has
                                          no such check); the next call that waits for the step returns
                                          VB200_ERR_NONFINITE naming the first bad element.  Off by default */
    int32_t step_kernel;               /* the whole step as ONE persistent kernel (one GPU, batch <= 64, widths up to
                                          64 x SMs/4, none of the optional stages): 0 = wherever that applies and
                                          gemm_path is AUTO, 1 = never, 2 = required (create fails otherwise) */
    int32_t dp_exchange;               /* VB200_DP_*: what volta_b200_dp_attach_peers switches the step to.  0 and 1:
                                          the peer-memory kernel.  2: copies; the arena then also holds one
                                          gradient-sized receive slot per rank, so it must be chosen at creation */
} vb200_config;

typedef struct vb200_handle vb200_handle;

/* volta_train_init(batch) -> Handle*  (mlp_train_rust_codegen.rs:641-667).
 * Allocates one device arena for the whole handle, initialises weights with the
 * reference's LCG-Xavier stream (seed 42, :630-638), biases zero, captures the step graph. */
int volta_b200_create(const vb200_config *cfg, vb200_handle **out);

/* volta_train_free (mlp_train_rust_codegen.rs:689-696). NULL is a no-op. */
void volta_b200_destroy(vb200_handle *h);

/* volta_train_step(h, X, Y, lr) (mlp_train_rust_codegen.rs:699-994).
 * X is [batch x L0], Y is [batch x Ln], row-major fp32; each may be a host pointer
 * (pageable or pinned; copied to the device inside the call) or a device pointer.
 * The call returns once X and Y have been consumed from host memory; the step itself
 * completes asynchronously on the handle's stream.  A host X of at least 64 MB travels in 2-8 row chunks
 * of at least 8192 rows, and the forward pass of a chunk starts as soon as it has landed, so that only the
 * first chunk's copy is exposed (VOLTA_B200_IN_CHUNKS=1 switches that off). */
int volta_b200_step(vb200_handle *h, const float *X, const float *Y, float lr);

/* volta_train_loss (mlp_train_rust_codegen.rs:686): loss of the last step (computed
 * before that step's update). Waits for the step to finish. */
float volta_b200_loss(vb200_handle *h);

/* volta_train_set_params(h, li, w, b) (mlp_train_rust_codegen.rs:670-675).
 * Host or device pointers; an out-of-range li is ignored, as in the reference. */
int volta_b200_set_params(vb200_handle *h, int32_t li, const float *w, const float *b);

/* volta_train_get_params(h, wo, bo) (mlp_train_rust_codegen.rs:678-684).
 * Fills wo[i], bo[i] (i < n layers) with pointers into a pinned host mirror owned by
 * the handle; the mirror is refreshed by this call (device -> host copy + wait) and
 * stays valid until destroy. */
int volta_b200_get_params(vb200_handle *h, float **wo, float **bo);

/* Forward pass only, with the handle's current weights: the GPU counterpart of the reference's
 * inference entry point volta_infer(in, in_n, out, out_n) (src/engine/ir/codegen/inner.rs:194-198),
 * which is compiled for batch 1 with the weights embedded.  Here in_n / L0 rows (at most the
 * handle's batch) go through the same fused GEMM + bias + activation kernels as training;
 * `in` and `out` may be host or device pointers; out_n must equal rows * Ln.  Call between steps. */
int volta_b200_infer(vb200_handle *h, const float *in, int64_t in_n, float *out, int64_t out_n);

/* LayerNorm scale and shift of hidden layer li (0 <= li < n-1), c = layers[li+1] floats each, host
 * pointers.  The reference keeps them inside the handle with no accessor (Handle fields ln_g/ln_b,
 * mlp_train_rust_codegen.rs:505-523); a checkpoint needs them.  Refused when use_layernorm is off. */
int volta_b200_get_layernorm(vb200_handle *h, int32_t li, float *gamma, float *beta);
int volta_b200_set_layernorm(vb200_handle *h, int32_t li, const float *gamma, const float *beta);

/* Test/diagnostic extensions (no counterpart in the reference): gradients of the
 * last step (same mirror convention), optimizer-state export/import for checkpoints
 * (the reference cannot export Adam moments, :670-684), and the Adam step counter.
 * The state is volta_b200_state_floats floats: first moments, second moments (as the
 * optimizer has them), then - with dropout on - two floats that carry the 64 raw bits of
 * the mask stream's position (copy them, do not do arithmetic on them). */
int volta_b200_get_grads(vb200_handle *h, float **dwo, float **dbo);
int64_t volta_b200_state_floats(vb200_handle *h);
int volta_b200_save_state(vb200_handle *h, float *out, int64_t n, uint64_t *step_out);
int volta_b200_load_state(vb200_handle *h, const float *in, int64_t n, uint64_t step);

/* Checkpoints in the reference's file formats (src/engine/model/checkpoint.rs): format 1 is the v1
 * text form (:14-44: header "#volta-checkpoint:v1", then "name|d0,d1|v0,v1,..." sorted by name; '#'
 * lines are comments), format 2 the v2 binary form (:162-213: magic "VOLTA\2\0\0" + a zlib stream of
 * stored blocks).  Files written here load in Volta's load_checkpoint / load_checkpoint_compressed and
 * the other way round.  One deviation: values are printed with nine SIGNIFICANT digits (every f32
 * survives), where the reference prints nine decimals (small values lose bits); both parse the other.
 * A vb200_checkpoint is a set of named fp32 tensors held on the host; it needs no GPU.
 * _load returns NULL on failure and volta_b200_last_error(NULL) says why (the reference's messages:
 * unsupported version, invalid format / shape / value at line N). */
typedef struct vb200_checkpoint vb200_checkpoint;
vb200_checkpoint *volta_b200_checkpoint_new(void);
void volta_b200_checkpoint_free(vb200_checkpoint *ck);
int volta_b200_checkpoint_add(vb200_checkpoint *ck, const char *name, const int64_t *shape, int32_t ndim,
                              const float *data);
/* format: 1 = v1 text (nine significant digits), 2 = v2 binary, 3 = v1 text with the reference's own
 * nine fixed decimals (byte-for-byte what save_checkpoint writes, checkpoint.rs:35; small values lose bits). */
int volta_b200_checkpoint_save(const vb200_checkpoint *ck, const char *path, int32_t format);
vb200_checkpoint *volta_b200_checkpoint_load(const char *path);
/* The same for the bytes of a checkpoint file held in memory (a file embedded in a library image). */
vb200_checkpoint *volta_b200_checkpoint_parse(const void *bytes, int64_t n);
/* Entry i in insertion order; the pointers stay valid until the next _add on, or the _free of, this checkpoint. */
int32_t volta_b200_checkpoint_count(const vb200_checkpoint *ck);
int volta_b200_checkpoint_entry(const vb200_checkpoint *ck, int32_t i, const char **name, const int64_t **shape,
                                int32_t *ndim, const float **data, int64_t *count);
/* Handle <-> checkpoint.  Names: "layer<i>.weight" [in, out], "layer<i>.bias" [out],
 * "layer<i>.ln_gamma/.ln_beta"; with_state adds the optimizer's moments ("layer<i>.weight.m", ".v",
 * ".acc" for Adagrad, ".mom" for SGD momentum; same for ".bias") and the counters "meta.adam_step",
 * "meta.dropout_rng" (three floats holding 22 + 22 + 20 bits each as exact integers) - what the
 * reference's checkpoint cannot carry (it stores parameters only).  Import takes every tensor it
 * knows by name, checks its shape, leaves the rest of the handle as it is and ignores other names.
 *
 * Volta names a layer's tensors after the layer ("{name}.weight", "{name}.bias" with the user's layer
 * names, src/engine/model/layers.rs:52-58).  The _named forms take one name per weight layer (a NULL
 * entry stands for "layer<i>") and use them instead of "layer<i>" for every tensor above.  Without
 * names, import looks for "layer<i>.*" first and otherwise takes the checkpoint's "<X>.weight" (2-D) +
 * "<X>.bias" pairs in sorted name order - the order Volta's writer uses - if there are exactly as many
 * as layers and every shape fits.  A checkpoint in which no parameter tensor is found is refused with
 * VB200_ERR_INVALID (it used to import nothing and report success); a found tensor of the wrong shape
 * likewise.  volta_b200_checkpoint_match runs the same name resolution without a handle or a GPU and
 * returns the number of parameter tensors found (> 0), or minus an error code with the reason in
 * volta_b200_last_error(NULL). */
int volta_b200_export_checkpoint(vb200_handle *h, vb200_checkpoint *ck, int32_t with_state);
int volta_b200_import_checkpoint(vb200_handle *h, const vb200_checkpoint *ck);
int volta_b200_export_checkpoint_named(vb200_handle *h, vb200_checkpoint *ck, int32_t with_state,
                                       const char *const *layer_names, int32_t n_names);
int volta_b200_import_checkpoint_named(vb200_handle *h, const vb200_checkpoint *ck, const char *const *layer_names,
                                       int32_t n_names);
int volta_b200_checkpoint_match(const vb200_config *cfg, const vb200_checkpoint *ck, const char *const *layer_names,
                                int32_t n_names);

/* Error reporting: last error code / message of this handle (or of the last failed
 * create when h is NULL).  The message pointer stays valid until the next call. */
int volta_b200_status(vb200_handle *h);
const char *volta_b200_last_error(vb200_handle *h);

/* The CUDA stream the handle launches on (a cudaStream_t), so that a harness can
 * record its own events on it; and a wait for everything queued on it. */
void *volta_b200_stream(vb200_handle *h);
int volta_b200_synchronize(vb200_handle *h);

/* Arena introspection: total bytes, and how many kernels one step launches
 * (graph nodes that are kernels, collectives excluded). */
int64_t volta_b200_arena_bytes(vb200_handle *h);
/* The memory plan of a configuration without creating anything (needs no GPU): total
 * arena bytes, the bytes it would take without reuse, and optionally one text line per
 * buffer, "name offset bytes first_use last_use persistent".  Mirrors what Volta's
 * memory planner reports (src/engine/ir/memory_planner.rs:47-144). */
int volta_b200_plan(const vb200_config *cfg, int64_t *arena_bytes, int64_t *unshared_bytes, char *report,
                    int64_t report_len);
int32_t volta_b200_kernels_per_step(vb200_handle *h);

/* Runs one step as plain launches with a CUDA event pair around every kernel and
 * returns up to `max` records: name (<= 47 chars), milliseconds, algorithmic flops and
 * bytes of that launch. Returns the number of records, or a negative error code.
 * Under NCCL data parallelism every rank must make the call (it is a step); the record
 * "wait_for_gradient_exchange" is then the part of the all-reduces that the backward GEMMs did
 * not hide.  Not available with the fused peer-memory exchange. */
typedef struct vb200_kernel_record {
    char name[48];
    float ms;
    double flops;
    double bytes;
} vb200_kernel_record;
int volta_b200_profile_step(vb200_handle *h, const float *X, const float *Y, float lr,
                            vb200_kernel_record *out, int32_t max);

/* Data-parallel bootstrap: rank 0 obtains an id and hands the same 128 bytes to every
 * rank's config (any host transport).  Uses NCCL, loaded at run time. */
int volta_b200_dp_unique_id(uint8_t out[128]);
/* Pre-flight check of that bootstrap, usable before any handle exists: joins a communicator of world_size
 * ranks as `rank`, sums `count` floats of device_buf over the ranks when count > 0 (every rank must make
 * the same call), and leaves the communicator again.  VB200_ERR_NCCL with NCCL's own message in
 * volta_b200_last_error(NULL) when any NCCL call fails (library missing, a rank count that does not
 * match, a system error).  $VOLTA_B200_NCCL_LIB selects the NCCL library file. */
int volta_b200_dp_check(const uint8_t id[128], int32_t world_size, int32_t rank, float *device_buf, int64_t count,
                        void *stream);

/* Fused data parallelism over peer memory (no counterpart in the reference).  After every rank has
 * created its handle (same configuration, world_size > 1), each exports the 64-byte IPC handle of its
 * arena; all ranks exchange them (any host transport) and attach the full list, ordered by rank.  From
 * then on a step no longer calls NCCL: per layer, one kernel per rank sums its share of every rank's
 * gradients with peer loads in rank order, applies the optimizer to that share and stores the new
 * parameters into every rank's arena; flag words in the arenas order the ranks, with bounded waits.
 * Needs peer access between the GPUs (NVLink); at most 8 ranks; optimizer state becomes sharded
 * (save_state is refused).
 * With dp_exchange = VB200_DP_PEER_COPY the attached handle exchanges by COPY instead: as soon as a layer's dW
 * exists, the rank's copy engines push it into its receive slot in every peer's arena (no SM is taken from the
 * backward GEMMs that run meanwhile); once a flag barrier shows that all ranks' pushes of the bucket have landed,
 * one kernel per rank adds the N copies in rank order and applies the optimizer to the whole bucket.  Every
 * rank keeps the full optimizer state (save_state works), and the sum has the same fixed order on every rank. */
int volta_b200_dp_ipc_handle(vb200_handle *h, uint8_t out[64]);
int volta_b200_dp_attach_peers(vb200_handle *h, const uint8_t *handles, int32_t count);
/* Failure detection of that path, checked without failing anything: runs ONE barrier kernel on this
 * handle alone with a declared world of `declared_world` ranks, every "peer" being the handle's own
 * arena, so that all flag words but its own are never written.  The kernel gives up after wait_ms,
 * sets the status bit and returns; the call then reports VB200_ERR_DEVICE_WAIT, the handle refuses
 * further steps and can still be queried and destroyed.  No counterpart in the reference (it has no
 * collective and no device-side wait). */
int volta_b200_dp_wait_selftest(vb200_handle *h, int32_t declared_world, int32_t wait_ms);

/* Stand-alone kernel entry points on device pointers (used by parity tests to check
 * single kernels against the oracle; `stream` is a cudaStream_t or NULL). */
int volta_b200_optimizer_apply(int32_t optimizer, float *p, float *s1, float *s2, const float *g, int64_t n,
                               int64_t n_decay, float lr, float weight_decay, float momentum, uint64_t t,
                               void *stream);
/* C[m x n] = op(A) . op(B): layout 0 = NN (A[m x k], B[k x n]), 1 = NT (A[m x k], B[n x k]),
 * 2 = TN (A[k x m], B[k x n]); path is VB200_GEMM_*. */
int volta_b200_gemm(int32_t layout, int32_t path, float *C, const float *A, const float *B, int64_t m,
                    int64_t n, int64_t k, void *stream);
/* Which kernel family a GEMM of this shape takes under `path`, and into how many K splits (a function of
 * the arguments alone; needs no GPU).  Returns VB200_ROUTE_* or minus an error code.  Operands are
 * assumed 16-byte aligned, as every buffer of a handle is. */
enum { VB200_ROUTE_FFMA = 0, VB200_ROUTE_TENSOR_SINGLE = 1, VB200_ROUTE_TENSOR_PAIR = 2, VB200_ROUTE_SMALL_ROWS = 3 };
int volta_b200_gemm_route(int32_t layout, int32_t path, int64_t m, int64_t n, int64_t k, int32_t *splits);
/* Self-check of the persistent step kernel's optimizer arithmetic (four elements side by side through
 * straight-line division / square-root cores, with a pre-check that sends a group with extreme operands to the
 * library routines) against the streaming optimizer's: `groups` seeded groups of four elements at Adam step t,
 * operands from the range training produces (wide = 0) or from all exponents (wide = 1).  counts[0] = elements
 * that differ in any bit of parameter or state (must be 0), [1] / [2] = groups that took the cores / the library
 * path.  optimizer: VB200_OPT_ADAM, _ADAMW or _ADAGRAD.  No counterpart in the reference. */
int volta_b200_update_selftest(int32_t optimizer, uint64_t seed, int64_t groups, int32_t wide, uint64_t t, uint64_t counts[3]);
/* out[j] = sum over rows of in[rows x cols] in a fixed order; scratch must hold
 * volta_b200_colsum_scratch_floats(rows, cols) floats. */
int64_t volta_b200_colsum_scratch_floats(int64_t rows, int64_t cols);
int volta_b200_colsum(float *out, const float *in, int64_t rows, int64_t cols, float *scratch, void *stream);

/* Column sums with NO allocation anywhere (no counterpart in the reference, which allocates
 * freely on the host): same result as volta_b200_colsum, bit for bit, but the scratch partials
 * live in a 4 MiB buffer built into the library image (1 Mi floats per GPU that loads the library,
 * held until process exit).  For callers that may not touch the CUDA allocator where they need a
 * bias gradient: latency-critical host threads that cannot take cudaMalloc's implicit
 * synchronisation, processes that have given all device memory to a pool of their own, plug-ins
 * whose host forbids allocation after start-up.  `out` [cols] and `in` [rows x cols] are the
 * caller's device buffers.  Inputs needing more than 1 Mi scratch floats
 * (volta_b200_colsum_scratch_floats says how many) are refused with VB200_ERR_TOO_LARGE and a
 * message on stderr.  The first call on each device looks up the buffer's device address; make
 * that call outside any stream capture.  All calls share the one buffer, which keeps whatever the
 * last call left (nothing in it needs to start at zero): two calls whose kernels can overlap on
 * the GPU - different streams without an ordering between them - race on it. */
int volta_b200_colsum_noalloc(float *out, const float *in, int64_t rows, int64_t cols, void *stream);

/* ---- Runtime-backend slice -------------------------------------------------------------------
 * What a `B200Backend` for Volta's runtime would bind (trait Backend, src/engine/ir/backend.rs:24-69):
 *   compile(plan)                      -> volta_b200_program_add per scheduled node + _compile
 *   execute_value / execute_terminal   -> _bind the context's inputs and parameters, _run, _fetch
 *   apply_gradients                    -> _update (parameters stay on the device between steps)
 * Nodes are added in schedule order (ExecutionPlan.schedule.ordered_nodes), each with the ValueId it
 * defines, the ValueIds it reads and its inferred shape (rank <= 2).  Op kinds mirror the variants of
 * the reference's Op enum that its MLP training graphs use (src/engine/ir/op.rs:40-135); semantics are
 * the interpreter's (src/engine/ir/interpreter.rs:680-880): numpy-style broadcasting for Add/Sub/Mul/Div,
 * the *Backward ops take (activation input, upstream gradient), Softmax runs over the last axis,
 * ReduceSum/ReduceMean carry attrs {axis (-1 = all), keepdims}, ConstTensor carries its data in attrs,
 * Reshape (same element count), Identity and Output share their operand's storage, SOFTMAX_XENT is
 * SoftmaxCrossEntropyLossFromLogits {logits, targets} -> scalar mean over the batch (interpreter.rs:776-815).
 * Everything else is refused with VB200_ERR_UNSUPPORTED.  Values that must stay readable after a run
 * (operands of Output nodes, gradients, anything fetched) are marked before compiling; other
 * temporaries share storage. */
enum { VB200_OP_INPUT = 0, VB200_OP_PARAMETER = 1, VB200_OP_CONST = 2, VB200_OP_ADD = 3, VB200_OP_SUB = 4,
       VB200_OP_MUL = 5, VB200_OP_DIV = 6, VB200_OP_NEG = 7, VB200_OP_TRANSPOSE = 8, VB200_OP_MATMUL = 9,
       VB200_OP_RELU = 10, VB200_OP_RELU_BACKWARD = 11, VB200_OP_SIGMOID = 12, VB200_OP_SIGMOID_BACKWARD = 13,
       VB200_OP_GELU = 14, VB200_OP_GELU_BACKWARD = 15, VB200_OP_SOFTMAX = 16, VB200_OP_LOG = 17, VB200_OP_EXP = 18,
       VB200_OP_REDUCE_SUM = 19, VB200_OP_REDUCE_MEAN = 20, VB200_OP_IDENTITY = 21, VB200_OP_OUTPUT = 22,
       VB200_OP_RESHAPE = 23, VB200_OP_SOFTMAX_XENT = 24 };

/* CompiledProgram (backend.rs:12-17) plus what the fused lowering did. */
typedef struct vb200_compiled_program {
    int64_t schedule_len;    /* nodes given */
    int64_t launches;        /* kernels the schedule became (Transpose folded into GEMM layouts, bias/activation
                                and activation-backward folded into GEMM epilogues when fuse != 0) */
    int64_t peak_bytes;      /* the arena */
    int64_t unshared_bytes;  /* what it would take without storage reuse */
    uint64_t fingerprint;    /* identity of the schedule (FNV-1a; not the reference's SipHash) */
} vb200_compiled_program;

/* OptimizerConfig (src/engine/ir/optimizer.rs:38-80); zero betas/eps/momentum select 0.9 / 0.999 / 1e-8 / 0.9. */
typedef struct vb200_optimizer_config {
    int32_t optimizer;       /* VB200_OPT_* */
    float lr, beta1, beta2, eps, weight_decay, momentum;
} vb200_optimizer_config;

typedef struct vb200_program vb200_program;
vb200_program *volta_b200_program_new(void);
void volta_b200_program_free(vb200_program *p);
const char *volta_b200_program_error(vb200_program *p);
int volta_b200_program_add(vb200_program *p, int32_t kind, int32_t value_id, const int32_t *inputs, int32_t n_inputs,
                           const int64_t *shape, int32_t ndim, const float *attrs, int32_t n_attrs);
int volta_b200_program_mark_output(vb200_program *p, int32_t value_id);
/* Plans the arena, lowers and captures the schedule; needs a GPU.  fuse = 0 keeps one kernel per node. */
int volta_b200_program_compile(vb200_program *p, int32_t fuse, vb200_compiled_program *info);
/* Inputs and parameters by ValueId (the ExecutionContext); host or device pointer, n floats.  A host buffer
 * is consumed before the call returns; a device buffer is copied on the program's stream and must stay
 * unchanged until the next _fetch (or any other call that waits for the program) has returned. */
int volta_b200_program_bind(vb200_program *p, int32_t value_id, const float *data, int64_t n);
int volta_b200_program_run(vb200_program *p);
int volta_b200_program_fetch(vb200_program *p, int32_t value_id, float *out, int64_t n);
/* apply_gradients (backend.rs:28-41; formulas of src/engine/ir/optimizer.rs:212-244, 329-340, 429-441,
 * 592-600): updates each parameter in place from its gradient value; moments live with the program.
 * `step` is the 1-based update count (Adam's bias corrections). */
int volta_b200_program_update(vb200_program *p, const vb200_optimizer_config *cfg, const int32_t *param_ids,
                              const int32_t *grad_ids, int32_t count, uint64_t step);

const char *volta_b200_version(void);
/* sizeof(vb200_config) as the library was built with: a binding checks its own mirror of the struct against it. */
int32_t volta_b200_config_size(void);

#ifdef __cplusplus
}
#endif
#endif /* VOLTA_B200_H */
