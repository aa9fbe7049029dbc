"""Parity of the tcgen05 kernels INSIDE training steps, at shapes where every GEMM family (forward with
bias + activation, dX with the activation derivative, dW) runs on them: the CTA-pair kernel, the single-CTA
kernel, K split over concurrent CTAs with the slab reduction applying the epilogue, ragged edges.

Arbiters: the C oracle with its GEMMs routed through the reference's own gemm_shim.c where that finishes in
seconds; tests/torch_fp64.py (pinned on the oracle) everywhere; and the library's own FFMA path, whose
per-element ascending-k sums are independent of tiling.  Bars as in test_gpu_parity.py: gradients within
1e-5 of the magnitude of the terms summed, weights after one step within 1e-5 of the tensor's largest weight
(plus the optimizer's response to the allowed gradient error), loss within 1e-3 (the achieved figures, far
smaller, are recorded through parity_report).  Bit identity: same bits from two fresh handles."""
import numpy as np
import pytest
import torch

from oracle.oracle import Oracle
from tests.test_gpu_parity import G_TOL, LOSS_TOL, W_TOL, update_fn
from tests.torch_fp64 import TorchMlp64
from volta_b200 import CONFIGS, TrainHandle, load_library, synth

pytestmark = pytest.mark.gpu

NN, NT, TN = 0, 1, 2
PATHS = {"auto": 0, "ffma": 1, "tensor": 2, "tensor_pair": 3}
ROUTE_NAMES = {0: "ffma", 1: "tensor_single", 2: "tensor_pair", 3: "small_rows"}


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def route(layout, path, m, n, k):
    import ctypes as C
    lib = load_library()
    s = C.c_int32(0)
    r = lib.volta_b200_gemm_route(layout, PATHS[path], m, n, k, C.byref(s))
    assert r >= 0
    return ROUTE_NAMES[r], int(s.value)


def step_routes(layers, B, path):
    """(family, splits) of every GEMM of one step, as the handle routes them."""
    out = {}
    for i, (r, c) in enumerate(zip(layers[:-1], layers[1:])):
        if c == 1:
            continue
        out["fwd%d" % i] = route(NN, path, B, c, r)
        out["dW%d" % i] = route(TN, path, r, c, B)
        if i > 0:
            out["dX%d" % i] = route(NT, path, B, r, c)
    return out


# ------------------------------------------------------------------------------- GEMM level
SPLIT_SHAPES = [
    # layout, path, m, n, k: the weight-gradient shape of the largest single-GPU configuration at a
    # quarter of its batch (256 pair tiles on 74 SM pairs), narrow outputs that split deeper, and the
    # single-CTA kernel's split
    (TN, "tensor_pair", 4096, 4096, 8192),
    (TN, "tensor_pair", 1024, 2048, 16384),
    (NN, "tensor_pair", 1024, 1024, 8192),
    (NT, "tensor_pair", 768, 1024, 8192),
    (TN, "tensor", 512, 1024, 16384),
    (NN, "tensor", 640, 384, 8192),
    (NT, "tensor", 1000, 260, 6144),
]


@pytest.mark.parametrize("layout,path,m,n,k", SPLIT_SHAPES)
def test_split_k_tensor_gemms_exact_on_integers_close_on_reals_and_repeatable(layout, path, m, n, k, parity_report):
    fam, splits = route(layout, path, m, n, k)
    assert fam.startswith("tensor") and splits > 1, (fam, splits)
    lib = load_library()
    rs = np.random.RandomState(m + 3 * n + 7 * k)

    def run(A, B):
        a_store = A if layout in (NN, NT) else np.ascontiguousarray(A.T)
        b_store = B if layout in (NN, TN) else np.ascontiguousarray(B.T)
        da, db = dev(a_store), dev(b_store)
        outs = []
        for _ in range(2):
            out = torch.full((m, n), float("nan"), device="cuda")
            assert lib.volta_b200_gemm(layout, PATHS[path], out.data_ptr(), da.data_ptr(), db.data_ptr(), m, n, k, None) == 0
            torch.cuda.synchronize()
            outs.append(out)
        assert torch.equal(outs[0], outs[1]), "same bits twice"
        return outs[0].cpu().numpy()

    # small integers: every product and every partial sum is exact in fp32, whatever the order
    Ai = rs.randint(-4, 5, size=(m, k)).astype(np.float32)
    Bi = rs.randint(-4, 5, size=(k, n)).astype(np.float32)
    want = (Ai.astype(np.float64) @ Bi.astype(np.float64)).astype(np.float32)
    assert np.array_equal(run(Ai, Bi), want)
    # reals against fp64, relative to |A|.|B|
    A = rs.randn(m, k).astype(np.float32)
    B = rs.randn(k, n).astype(np.float32)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64)
    err = float(np.max(np.abs(run(A, B).astype(np.float64) - ref) / bound))
    parity_report("gemm_splitk", layout=layout, path=fam, m=m, n=n, k=k, splits=splits, max_err_over_absA_absB=err)
    assert err <= 2e-6


# ------------------------------------------------------------------------------- step level
def weights_and_inputs(layers, B, x_dist="normal"):
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    rs = np.random.RandomState(5)
    bs = [(rs.randn(*b.shape) * 0.05).astype(np.float32) for b in bs]
    x = synth.rows(x_dist, 1234, 0, B, layers[0])
    y = synth.rows("normal", 4321, 0, B, layers[-1])
    return ws, bs, x, y


def make_handle(layers, act, opt, B, path, ws, bs):
    g = TrainHandle(layers, act, opt, B, gemm_path=path)
    for i, (w, b) in enumerate(zip(ws, bs)):
        g.set_params(i, w, b)
    return g


def compare_step(g, ref_grads, ref_params, ref_loss, scales, opt, lr, s1, s2, t, label, parity_report, fragile=None,
                 robust=False, **info):
    """One step from identical state: gradients, loss and weights of handle g against a reference given as flat
    lists (weights then biases).  Records the achieved errors, then applies the bars.

    `fragile` = (columns per hidden layer, count) from TorchMlp64.fragile_units(): hidden units of a relu network
    whose pre-activation is below fp32 resolution, so that two correct fp32 evaluations may disagree on their
    derivative.  Such a unit's own gradient column (dW_i[:, j], db_i[j]) is then left out of the comparison, and
    every flip may move the other gradients by a few 1e-5 of their scale (one batch row's share of the sum), so the
    gradient bar is widened to 1e-5 * (1 + 3 * count).

    Weights: every element within 1e-5 of the tensor's largest weight plus the optimizer's response to the allowed
    gradient error.  Only elements whose gradient is itself no larger than ten times that allowed error can need the
    second term (Adam and Adagrad divide by a running magnitude of the gradient, so there the update is sign-like);
    the number of elements beyond the plain 1e-5 is held to their number.

    robust = True is for relu networks so large that thousands of units are fragile (the derivative is
    discontinuous: per-element bars are then ill-posed in any fp32 arithmetic, the reference's included): the
    gradients are held only to 1e-2 (of their scale at the worst element, and in the root-mean-square sense of the
    rms gradient per tensor: a flipped unit changes one whole gradient column), the loss as always, and the
    per-element weight bars are not applied.  The same network with a smooth activation is held to every bar."""
    n = len(ref_grads) // 2
    frag_cols, frag_count = fragile if fragile is not None else ([np.zeros(0, np.int64)] * (n - 1), 0)
    g_tol = G_TOL["auto"] * (1.0 + 3.0 * frag_count)

    def keep_mask(idx, shape):
        """False where tensor idx (weights 0..n-1, then biases) belongs to a fragile unit's own column."""
        layer = idx % n
        keep = np.ones(shape, bool)
        if layer < n - 1 and len(frag_cols[layer]):
            keep[..., frag_cols[layer]] = False
        return keep

    gdw, gdb = g.get_grads()
    g_err, g_rms = 0.0, 0.0
    for idx, (a, b, sc) in enumerate(zip(gdw + gdb, ref_grads, scales)):
        err = np.abs(a.astype(np.float64) - b)
        g_rms = max(g_rms, float(np.sqrt(np.mean(err * err)) / max(np.sqrt(np.mean(np.square(b))), 1e-300)))
        err = err[keep_mask(idx, err.shape)]
        if err.size:
            g_err = max(g_err, float(np.max(err)) / sc)
    w_err, beyond, total, w_ok, ill = 0.0, 0, 0, True, 0
    for idx, (a, b, gr, sc, m1, m2) in enumerate(zip(sum(g.get_params(), []), ref_params, ref_grads, scales, s1, s2)):
        wmax = float(np.max(np.abs(b)))
        keep = keep_mask(idx, b.shape)
        diff = np.abs(a.astype(np.float64) - b)
        w_err = max(w_err, float(np.max(diff[keep])) / max(wmax, 1e-30) if keep.any() else 0.0)
        tol = np.full(b.shape, W_TOL * wmax, np.float64)
        u = update_fn(opt, lr, m1, m2, t)
        d = g_tol * sc
        gr = gr.astype(np.float64)
        tol += np.maximum(np.abs(u(gr + d) - u(gr)), np.abs(u(gr - d) - u(gr)))
        w_ok = w_ok and bool(np.all(diff[keep] <= tol[keep]))
        beyond += int(np.sum(diff[keep] > W_TOL * wmax))
        ill += int(np.sum(np.abs(gr[keep]) <= 10.0 * d))
        total += int(keep.sum())
    loss_err = abs(g.loss() - ref_loss) / abs(ref_loss)
    parity_report("step", against=label, grad_err_over_scale=g_err, grad_rms_err_over_rms=g_rms, weight_rel_err=w_err,
                  loss_rel_err=loss_err, weights_beyond_1e5=beyond, weights_with_gradient_near_its_error_bar=ill,
                  weights=total, fragile_units=frag_count, robust=robust, **info)
    assert loss_err <= LOSS_TOL, "%s: loss" % label
    if robust:
        assert g_rms <= 1e-2, "%s: gradients, rms (%g of the rms gradient)" % (label, g_rms)
        assert g_err <= 1e-2, "%s: gradients (%g of their scale)" % (label, g_err)
        return g_err, w_err, loss_err
    assert g_err <= g_tol, "%s: gradients (%g of their scale, bar %g)" % (label, g_err, g_tol)
    assert w_ok, "%s: weights after one step" % label
    assert beyond <= ill, "%s: %d weights beyond the plain bar, %d ill-conditioned" % (label, beyond, ill)
    return g_err, w_err, loss_err


STEP_CASES = [
    # layers, activation, optimizer, batch, path.  2304 = 9 pair tiles a side (two bands of the tile walk, more
    # than one wave of the 74 SM pairs).  Alternating 1536/2304 widths give, in ONE step, pair-kernel GEMMs that
    # apply their epilogue themselves (K = 1536: bias + SiLU with two outputs, the activation derivative) and
    # ones that split K and leave it to the slab reduction (K = 2304).  2300/2308 leave ragged edges in every
    # dimension; silu/gelu keep the pre-activation; width-one output as in the benchmark models.
    ([1536, 2304, 1536, 2304], "silu", "sgd_momentum", 2304, "tensor_pair"),
    ([2300, 2308, 2300, 1], "gelu", "adam", 1540, "tensor_pair"),
    ([768, 1024, 768, 8], "relu", "adamw", 1024, "tensor_pair"),
    ([2304, 2304, 2304, 2304], "silu", "sgd_momentum", 2304, "auto"),
    ([1000, 1028, 516, 4], "tanh", "adagrad", 1100, "tensor"),
]


@pytest.mark.parametrize("layers,act,opt,B,path", STEP_CASES)
def test_steps_on_the_tensor_kernels_match_fp64_the_ffma_path_and_repeat_bit_for_bit(layers, act, opt, B, path,
                                                                                       parity_report):
    routes = step_routes(layers, B, path)
    assert all(f.startswith("tensor") for f, _ in routes.values()), routes
    if path == "tensor_pair":
        # every GEMM whose output is at least 256 x 256 is on the pair kernel, and for each family at least one
        # of them unsplit, so that the kernel's own fused epilogue runs
        wide = {k: v for k, v in routes.items() if not (k.endswith(str(len(layers) - 2)) and layers[-1] < 256)}
        assert all(f == "tensor_pair" for f, _ in wide.values()), routes
        if layers == STEP_CASES[0][0]:   # built so that every family has both an unsplit and a split pair GEMM
            for fam in ("fwd", "dW", "dX"):
                assert any(k.startswith(fam) and v == ("tensor_pair", 1) for k, v in routes.items()), (fam, routes)
    lr = 1e-3 if opt in ("adam", "adamw") else 1e-2
    ws, bs, x, y = weights_and_inputs(layers, B)
    t64 = TorchMlp64(layers, act, opt, ws, bs)
    s1, s2, t0 = t64.state_before_lists()
    t64.step(x, y, lr)
    scales = t64.gradient_scales()
    info = dict(layers=layers, activation=act, optimizer=opt, batch=B, path=path,
                routes=sorted(set("%s/s%d" % r for r in routes.values())))

    g = make_handle(layers, act, opt, B, path, ws, bs)
    g.step(x, y, lr)
    fragile = t64.fragile_units()
    compare_step(g, t64.grads(), t64.params(), t64.loss(), scales, opt, lr, s1, s2, t0 + 1, "torch fp64", parity_report,
                 fragile=fragile, **info)
    # the library's FFMA path from the same state (fp32, ascending k per element)
    f = make_handle(layers, act, opt, B, "ffma", ws, bs)
    f.step(x, y, lr)
    fgrads = [a.astype(np.float64) for a in sum(f.get_grads(), [])]
    fparams = [a.astype(np.float64) for a in sum(f.get_params(), [])]
    compare_step(g, fgrads, fparams, f.loss(), scales, opt, lr, s1, s2, t0 + 1, "own ffma path", parity_report,
                 fragile=fragile, **info)
    f.free()
    # second step (state now non-trivial), then bit identity against a fresh handle
    t64.step(x, y, lr)
    g.step(x, y, lr)
    assert abs(g.loss() - t64.loss()) <= LOSS_TOL * abs(t64.loss())
    h2 = make_handle(layers, act, opt, B, path, ws, bs)
    for _ in range(2):
        h2.step(x, y, lr)
    assert np.float32(g.loss()).view(np.uint32) == np.float32(h2.loss()).view(np.uint32)
    for a, b in zip(sum(g.get_params(), []), sum(h2.get_params(), [])):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    g.free()
    h2.free()


def test_pair_kernel_step_matches_the_oracle_on_the_references_own_gemm(parity_report):
    """The same comparison against the C restatement of the step with every GEMM computed by the reference's
    gemm_shim.c (compiled unmodified): fp32 against fp32, two steps, SiLU + momentum as in the largest
    single-GPU configuration."""
    layers, act, opt, B, lr = [1024, 1280, 1024, 1], "silu", "sgd_momentum", 1024, 1e-2
    ws, bs, x, y = weights_and_inputs(layers, B, "uniform")
    o = Oracle(layers, act, opt, B)
    if o.use_reference_gemm() is None:
        pytest.skip("no prebuilt reference GEMM shim fits this CPU")
    for i, (w, b) in enumerate(zip(ws, bs)):
        o.set_params(i, w, b)
    g = make_handle(layers, act, opt, B, "tensor_pair", ws, bs)
    routes = step_routes(layers, B, "tensor_pair")
    assert all(f == "tensor_pair" for f, _ in routes.values()), routes
    t64 = TorchMlp64(layers, act, opt, ws, bs)
    for step in range(2):
        s1w, s1b, s2w, s2b, t_prev = o.state()
        zeros = lambda ref: [np.zeros_like(p) for p in ref]
        ref_p = sum(o.get_params(), [])
        s1 = [a if a is not None else z for a, z in zip(s1w + s1b, zeros(ref_p))]
        s2 = [a if a is not None else z for a, z in zip(s2w + s2b, zeros(ref_p))]
        o.step(x, y, lr)
        t64.step(x, y, lr)
        g.step(x, y, lr)
        compare_step(g, [a.astype(np.float64) for a in sum(o.get_grads(), [])],
                     [a.astype(np.float64) for a in sum(o.get_params(), [])], o.loss(), t64.gradient_scales(), opt, lr,
                     s1, s2, t_prev + 1, "oracle + reference gemm_shim.c, step %d" % (step + 1), parity_report,
                     fragile=t64.fragile_units(),
                     layers=layers, activation=act, optimizer=opt, batch=B, path="tensor_pair")
    g.free()


# ------------------------------------------------------------------- the large configurations
def run_config_against_fp64(cfg, B, steps, parity_report, path="auto", also_oracle=False, robust=False):
    """First step against fp64 at the one-step bars; then the free run.  The stated bar for the loss after the
    configuration's step count is 1e-3.  Adam-type trajectories amplify any admissible difference (their update is
    sign-like where a gradient is near zero), so that bar is applied modulo the trajectory's own sensitivity: a
    twin fp64 run whose weights are moved after the first step by the amount the one-step bar allows (1e-5 of each
    tensor's largest weight, random signs) shows how far the final loss moves for an error of admissible size; the
    reference's own fp32 arithmetic (the oracle on its gemm_shim.c) shows the same kind of drift.  With the oracle
    at hand the last state is also teacher-forced: one step from the oracle's exact state at the one-step bars."""
    layers = list(cfg.layers)
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    x = synth.rows(cfg.x_dist, 1234, 0, B, layers[0])
    y = synth.rows(cfg.y_dist, 4321, 0, B, layers[-1])
    g = make_handle(layers, cfg.activation, cfg.optimizer, B, path, ws, bs)
    t64 = TorchMlp64(layers, cfg.activation, cfg.optimizer, ws, bs)
    twin = TorchMlp64(layers, cfg.activation, cfg.optimizer, ws, bs) if steps > 1 else None
    o = None
    if also_oracle:
        o = Oracle(layers, cfg.activation, cfg.optimizer, B)
        if o.use_reference_gemm() is None:
            o = None
        else:
            for i, (w, b) in enumerate(zip(ws, bs)):
                o.set_params(i, w, b)
    routes = step_routes(layers, B, path)
    info = dict(config=cfg.name, batch=B, steps=steps, path=path, routes=sorted(set("%s/s%d" % r for r in routes.values())))
    for step in range(steps):
        if step == 0:
            s1, s2, t0 = t64.state_before_lists()
        t64.step(x, y, cfg.lr)
        g.step(x, y, cfg.lr)
        if twin is not None:
            twin.step(x, y, cfg.lr)
        if o is not None:
            o.step(x, y, cfg.lr)
        if step == 0:
            compare_step(g, t64.grads(), t64.params(), t64.loss(), t64.gradient_scales(), cfg.optimizer, cfg.lr, s1, s2,
                         t0 + 1, "torch fp64, first step", parity_report, fragile=t64.fragile_units(), robust=robust, **info)
            if twin is not None:
                gen = torch.Generator().manual_seed(7)
                for p in twin.w + twin.b:
                    p += (torch.rand(p.shape, generator=gen, dtype=torch.float64) * 2.0 - 1.0) * (W_TOL * float(p.abs().max()))
    lg, l64 = g.loss(), t64.loss()
    lo = o.loss() if o is not None else None
    sens = abs(twin.loss() - l64) if twin is not None else 0.0
    parity_report("config_run", gpu_loss=lg, fp64_loss=l64, oracle_f32_loss=lo, loss_rel_err_vs_fp64=abs(lg - l64) / abs(l64),
                  oracle_f32_vs_fp64=(abs(lo - l64) / abs(l64) if lo is not None else None),
                  sensitivity_to_admissible_one_step_error=sens / abs(l64), **info)
    # a chaotic quantity: the allowance is three times the larger of the two drifts seen from admissible causes
    # (the twin's, and that of the reference's own fp32 arithmetic where it was run)
    drift = max(sens, abs(lo - l64) if lo is not None else 0.0)
    allowed = max(LOSS_TOL * abs(l64), 3.0 * drift)
    assert abs(lg - l64) <= allowed, "loss after %d steps: gpu %g, fp64 %g, oracle fp32 %s, allowed %g" % (steps, lg, l64, lo, allowed)
    if o is not None:
        # and pinned along the real trajectory: the handle takes ONE more step from the fp32 oracle's exact
        # parameters and optimizer state, which must agree with the oracle's next step at the one-step bars
        from tests.test_gpu_parity import assert_one_step_parity, sync_gpu_to_oracle
        sync_gpu_to_oracle(g, o)
        before = o.state()
        g.step(x, y, cfg.lr)
        o.step(x, y, cfg.lr)
        assert_one_step_parity(g, o, cfg.optimizer, cfg.lr, before)
    g.free()
    return routes


def test_c3_at_batch_1024_for_its_fifty_steps(parity_report):
    """Configuration 3 at its stated batch and step count (GELU, AdamW; every GEMM on the tensor kernels)."""
    routes = run_config_against_fp64(CONFIGS["c3_b1024"], 1024, 50, parity_report, also_oracle=True)
    assert all(f.startswith("tensor") for f, _ in routes.values()), routes


def test_c4_topology_at_batch_8192(parity_report):
    """Configuration 4's widths at an eighth of its batch (its per-GPU batch on eight GPUs): the pair kernel
    with all three epilogues and the weight-gradient GEMMs that split K inside the step (slabs in the arena,
    epilogue in the slab reduction)."""
    routes = run_config_against_fp64(CONFIGS["c4"], 8192, 2, parity_report)
    assert all(f == "tensor_pair" for f, _ in routes.values()), routes
    assert any(s > 1 for _, s in routes.values()), routes


def test_c5_topology_at_batch_512(parity_report):
    """Configuration 5's widths (402.7 M parameters, Adam) at a reduced batch; one step against fp64.  Twice: with
    a smooth activation in place of relu, where every per-element bar applies and pins the kernels at these widths
    (K split four ways among them); and as specified, with relu, where some thousands of the 18.9 M hidden units
    sit within fp32 noise of zero and the comparison is the robust one (see compare_step)."""
    import dataclasses
    smooth = dataclasses.replace(CONFIGS["c5"], name="c5_silu", activation="silu")
    routes = run_config_against_fp64(smooth, 512, 1, parity_report)
    assert all(f.startswith("tensor") for f, _ in routes.values()), routes
    assert any(s > 1 for _, s in routes.values()), routes
    run_config_against_fp64(CONFIGS["c5"], 512, 1, parity_report, robust=True)


@pytest.mark.parametrize("name,B", [("c4", 8192), ("c3_b1024", 1024)])
def test_large_configurations_repeat_bit_for_bit(name, B):
    cfg = CONFIGS[name]
    layers = list(cfg.layers)
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    x = synth.rows(cfg.x_dist, 1234, 0, B, layers[0])
    y = synth.rows(cfg.y_dist, 4321, 0, B, layers[-1])
    runs = []
    for _ in range(2):
        g = make_handle(layers, cfg.activation, cfg.optimizer, B, "auto", ws, bs)
        losses = []
        for _ in range(4):
            g.step(x, y, cfg.lr)
            losses.append(np.float32(g.loss()).view(np.uint32))
        runs.append((losses, [p.view(np.uint32).copy() for p in sum(g.get_params(), [])]))
        g.free()
    assert runs[0][0] == runs[1][0]
    for a, b in zip(runs[0][1], runs[1][1]):
        assert np.array_equal(a, b)
