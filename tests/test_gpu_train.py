"""GPU training step (cross-entropy + Adam) against the reference-made golden gradients / Adam
trajectory and against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest

import nets
from conftest import golden

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(has_gpu):
    assert has_gpu, "no CUDA device"


def _flat(c, wfield, bfield):
    return np.concatenate([np.ctypeslib.as_array(getattr(c, wfield), shape=(c.total_weights,)),
                           np.ctypeslib.as_array(getattr(c, bfield), shape=(c.total_biases,))]).copy()


def test_one_full_batch_step_matches_reference_gradients(spg, oracle):
    """net->grad_* after one train() step equal the reference's batch gradients (golden), and the
    updated weights equal oracle gradients + oracle Adam."""
    g = np.load(golden("train.npz"))
    net = spg.Network.load(golden("train.fp32.nn"))
    onet = oracle.OracleNet.from_file(golden("train.fp32.nn"))
    w0 = np.concatenate([net.weights, net.biases]).copy()
    net.train(g["x"], g["t"], epochs=1, strategy=spg.abi.STRATEGY_FULL_BATCH, learning_rate=1e-3)
    grads = _flat(net.c, "grad_weights", "grad_biases")
    ref = g["grads"]
    assert np.linalg.norm(grads - ref) / np.linalg.norm(ref) <= 1e-5
    assert net.c.time_step == 1
    # first Adam step from zero state: factors as train() forms them (Training.c:480-482, :777-779)
    w, m, v = w0.copy(), np.zeros_like(w0), np.zeros_like(w0)
    fp = C.POINTER(C.c_float)
    og = onet.gradients(g["x"], g["t"], 1.0 / g["x"].shape[0])
    mf = np.float32(1.0) / (np.float32(1.0) - np.float32(0.9))
    vf = np.float32(1.0) / (np.float32(1.0) - np.float32(0.999))
    oracle.Oracle.lib().spgo_adam(w.ctypes.data_as(fp), m.ctypes.data_as(fp), v.ctypes.data_as(fp), og.ctypes.data_as(fp),
                                  w.size, 1e-3, 0.9, 0.999, mf, vf, 1e-8)
    got = np.concatenate([net.weights, net.biases])
    # the first Adam step is lr*sign(g) wherever |g| >> sqrt(eps): compare where the gradient is not ~0
    solid = np.abs(og) > 1e-6
    assert np.abs(got - w)[solid].max() <= 2e-6
    assert np.abs(_flat(net.c, "opt_m_weights", "opt_m_biases") - m).max() <= 1e-7
    net.free()


def test_adam_kernel_matches_reference_trajectory(spg):
    import torch
    g = np.load(golden("train.npz"))
    lib = spg.lib()
    lib.spgk_adam.argtypes = [C.c_void_p] * 4 + [C.c_uint64] + [C.c_float] * 7 + [C.c_void_p]
    w = torch.from_numpy(g["adam_w0"].copy()).cuda()
    m, v = torch.zeros_like(w), torch.zeros_like(w)
    b1p = b2p = np.float32(1.0)
    for step in range(10):
        b1p = np.float32(b1p * np.float32(0.9))
        b2p = np.float32(b2p * np.float32(0.999))
        mf = np.float32(1.0) / (np.float32(1.0) - b1p)
        vf = np.float32(1.0) / (np.float32(1.0) - b2p)
        gs = torch.from_numpy(g["adam_g"][step].copy()).cuda()
        assert lib.spgk_adam(w.data_ptr(), m.data_ptr(), v.data_ptr(), gs.data_ptr(), w.numel(),
                             1e-3, 0.9, 0.999, float(mf), float(vf), 1e-8, 1.0, None) == 0
        assert np.abs(w.cpu().numpy() - g["adam_w"][step]).max() <= 1e-6
    assert np.abs(m.cpu().numpy() - g["adam_m"]).max() <= 1e-7 and np.abs(v.cpu().numpy() - g["adam_v"]).max() <= 1e-8


def test_minibatch_training_reduces_loss_on_the_benchmark_mlp(spg, oracle):
    """784-512-1000-10, He init, 256-row mini-batches, Adam lr 1e-3, uniform one-hot targets:
    the cross-entropy reported through the callback falls, and the trained weights serve inference."""
    net = spg.Network.build(nets.A_TOPO, nets.A_ACTS, spg.abi.WEIGHT_INITIALIZATION_HE, seed=5)
    rng = np.random.default_rng(0)
    n = 1024
    x = rng.random((n, 784), dtype=np.float32)
    t = np.zeros((n, 10), np.float32)
    t[np.arange(n), rng.integers(0, 10, n)] = 1.0
    errors = []
    spg.lib().spingalett_seed(9)
    net.train(x, t, epochs=30, batch_size=256, strategy=spg.abi.STRATEGY_SMALL_BATCH, learning_rate=1e-3,
              callback=lambda h, epoch, err: errors.append(err) or False, callback_interval=1, nan_check_interval=10)
    assert len(errors) == 30 and net.c.time_step == 30 * 4
    assert errors[0] > 2.0 and errors[-1] < 0.5 * errors[0], errors
    assert np.all(np.isfinite(net.weights))
    # inference afterwards runs on the trained weights (device image refreshed) and matches the oracle on them
    onet = oracle.OracleNet.from_arrays(net.topology, net.acts, net.weights, net.biases)
    spg.set_math_mode(spg.abi.MATH_EXACT)
    got = net.forward_batch(x[:64])
    assert np.abs(got - onet.forward_batch(x[:64])).max() <= 2e-5
    spg.set_math_mode(spg.abi.MATH_AUTO)
    acc = np.mean(np.argmax(net.forward_batch(x), 1) == np.argmax(t, 1))
    assert acc > 0.5
    net.free()


def test_sigmoid_output_and_ragged_last_batch(spg, oracle):
    """Cross-entropy over a sigmoid output layer, batch size that does not divide the sample count."""
    net = spg.Network.build([12, 9, 3], [spg.abi.ACT_FOO52, spg.abi.ACT_SIGMOID], spg.abi.WEIGHT_INITIALIZATION_HE, seed=4)
    onet = oracle.OracleNet.from_arrays(net.topology, net.acts, net.weights, net.biases)
    rng = np.random.default_rng(1)
    x = rng.random((10, 12), dtype=np.float32)
    t = (rng.random((10, 3)) > 0.5).astype(np.float32)
    net.train(x, t, epochs=1, strategy=spg.abi.STRATEGY_FULL_BATCH, learning_rate=1e-2)
    grads = _flat(net.c, "grad_weights", "grad_biases")
    og = onet.gradients(x, t, 0.1)
    assert np.linalg.norm(grads - og) / np.linalg.norm(og) <= 1e-5
    net.train(x, t, epochs=2, batch_size=4, strategy=spg.abi.STRATEGY_SMALL_BATCH)      # batches of 4, 4, 2
    assert net.c.time_step == 1 + 2 * 3
    net.free()


@pytest.mark.parametrize("outw,act", [(24, "softmax"), (20, "sigmoid"), (7, "softmax")])
def test_wide_and_narrow_output_layers_match_oracle_gradients(spg, oracle, outw, act):
    """An output layer of more than 16 units takes product + softmax rows + delta kernel, a narrower one the one-launch
    output kernel: both give the oracle's gradients, and the loss that train() reports is finite."""
    out_act = spg.abi.ACT_SOFTMAX if act == "softmax" else spg.abi.ACT_SIGMOID
    net = spg.Network.build([16, 40, outw], [spg.abi.ACT_RELU, out_act], spg.abi.WEIGHT_INITIALIZATION_HE, seed=11)
    onet = oracle.OracleNet.from_arrays(net.topology, net.acts, net.weights, net.biases)
    rng = np.random.default_rng(outw)
    x = rng.random((48, 16), dtype=np.float32)
    if act == "softmax":
        t = np.zeros((48, outw), np.float32)
        t[np.arange(48), rng.integers(0, outw, 48)] = 1.0
    else:
        t = (rng.random((48, outw)) > 0.5).astype(np.float32)
    net.train(x, t, epochs=1, strategy=spg.abi.STRATEGY_FULL_BATCH, learning_rate=1e-3)
    grads = _flat(net.c, "grad_weights", "grad_biases")
    og = onet.gradients(x, t, 1.0 / 48)
    assert np.linalg.norm(grads - og) / np.linalg.norm(og) <= 1e-5
    net.free()


def test_invalid_training_requests_are_refused(spg):
    lib, a = spg.lib(), spg.abi
    net = spg.Network.build([4, 3, 2], [a.ACT_RELU, a.ACT_SOFTMAX], a.WEIGHT_INITIALIZATION_HE, seed=1)
    x = np.zeros((4, 4), np.float32)
    t = np.zeros((4, 2), np.float32)
    with pytest.raises(spg.SpingalettError):
        net.train(x, t, epochs=0)
    with pytest.raises(spg.SpingalettError) as e:
        net.train(x, t, epochs=1, optimizer=17)
    assert e.value.code == a.ERR_INVALID
    hidden = spg.Network.build([4, 3, 2], [a.ACT_SOFTMAX, a.ACT_SOFTMAX], a.WEIGHT_INITIALIZATION_HE, seed=1)
    with pytest.raises(spg.SpingalettError) as e:                                      # Training.c:620-626
        hidden.train(x, t, epochs=1, strategy=a.STRATEGY_FULL_BATCH)
    assert "hidden" in str(e.value)
    for n in (net, hidden):
        n.free()


def _train_case_names():
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(os.path.dirname(golden("x")), "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.TRAIN_CASES


@pytest.mark.parametrize("case", _train_case_names(), ids=lambda c: c[0])
def test_every_update_rule_and_output_delta_matches_the_reference_run(spg, case):
    """SGD / MOMENTUM / RMSPROP / ADAM / ADAMW with weight decay, global-norm clipping, MSE and MSE+softmax deltas, cross-entropy
    over a non-softmax output, and per-sample training: final parameters and reported loss against the reference's own
    train() on the same net and batch (tests/golden/train_surface.npz)."""
    name, strat, opt, loss, out_act, decay, clip, epochs, batch = case
    g, ref = np.load(golden("train.npz")), np.load(golden("train_surface.npz"))
    net = spg.Network.load(golden("train.fp32.nn"))
    c = net.c
    c.act_func[c.layers - 2] = out_act
    c.loss_func = loss
    seen = {}

    def cb(_net, epoch, err):
        seen["loss"] = float(err)
        seen["epochs"] = epoch
        return False
    net.train(g["x"], g["t"], epochs=epochs, batch_size=batch, strategy=strat, optimizer=opt, learning_rate=0.01,
              weight_decay=decay, max_grad_norm=clip, callback=cb, callback_interval=1)
    w, b = net.weights.copy(), net.biases.copy()
    rw, rb = ref[name + ".w"], ref[name + ".b"]
    # Adam-like rules move every weight by about lr per step whatever the gradient's size, so where a gradient is ~0 the
    # summation order decides its sign; those few elements are judged by the norm, the rest element by element
    tol = 2e-5 if opt in (spg.abi.OPTIMIZER_SGD, spg.abi.OPTIMIZER_MOMENTUM) else 2e-3
    err = np.abs(np.concatenate([w - rw, b - rb]))
    assert np.linalg.norm(err) <= 1e-3 * np.linalg.norm(np.concatenate([rw, rb])), (name, err.max())
    assert np.quantile(err, 0.98) <= tol and err.max() <= 0.05, (name, err.max(), np.quantile(err, 0.98))
    assert seen["epochs"] == epochs
    assert abs(seen["loss"] - float(ref[name + ".loss"])) <= 2e-4 * max(1.0, abs(float(ref[name + ".loss"]))), (name, seen["loss"])
    assert net.c.time_step == (epochs * g["x"].shape[0] if strat == spg.abi.STRATEGY_SAMPLE else epochs)
    net.free()


def test_autosave_writes_the_device_state_and_state_survives_calls(spg, oracle, tmp_path):
    """AUTOSAVE_NEW_FILES / AUTOSAVE_OVERWRITE (Training.c:536-578): files named like the reference's, written from the
    trainer's device buffers while train() runs; the last one equals what the net holds afterwards.  A second train() call
    on the same net reuses the device state of the first."""
    a = spg.abi
    g = np.load(golden("train.npz"))
    net = spg.Network.load(golden("train.fp32.nn"))
    base = str(tmp_path / "ckpt.nn")
    net.train(g["x"], g["t"], epochs=4, strategy=a.STRATEGY_FULL_BATCH, learning_rate=0.01, autosave_mode=2, autosave_interval=2,
              autosave_path=base)                                                       # AUTOSAVE_NEW_FILES
    names = sorted(p.name for p in tmp_path.iterdir())
    assert names == ["ckpt_epoch_2.nn", "ckpt_epoch_4.nn"], names
    last = oracle.OracleNet.from_file(str(tmp_path / "ckpt_epoch_4.nn"))
    assert last.has_optimizer and last.time_step == 4
    assert np.array_equal(last.weights, net.weights) and np.array_equal(last.biases, net.biases)
    mid = oracle.OracleNet.from_file(str(tmp_path / "ckpt_epoch_2.nn"))
    assert mid.time_step == 2 and not np.array_equal(mid.weights, net.weights)
    # overwrite mode, quantised, without optimizer sections; then a second call on the same net
    one = str(tmp_path / "one")
    net.train(g["x"], g["t"], epochs=3, strategy=a.STRATEGY_FULL_BATCH, learning_rate=0.01, autosave_mode=1, autosave_interval=1,
              autosave_path=one, autosave_precision=a.PRECISION_INT8, autosave_with_optimizer=False)   # AUTOSAVE_OVERWRITE
    q = oracle.OracleNet.from_file(one + ".nn")                                          # ".nn" appended as save does
    assert q.precision == a.PRECISION_INT8 and not q.has_optimizer and net.c.time_step == 7
    want = oracle.Oracle.decode(oracle.Oracle.encode(net.weights[: 12 * 16], a.PRECISION_INT8), 12 * 16, a.PRECISION_INT8)
    assert np.array_equal(q.weights[: 12 * 16], want)
    net.free()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_two_rank_data_parallel_step(spg, tmp_path, world):
    """`world` processes, one GPU each, through both gradient exchanges (the one-kernel exchange over peer memory and the
    NCCL all-reduce): the summed gradient equals the gradient of the concatenated batch, and weights, gradients and
    optimiser moments end bit-identical on every rank.  Needs `world` GPUs."""
    if spg.lib().spingalett_get_device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import os
    import subprocess
    import sys
    worker = os.path.join(os.path.dirname(__file__), "dist_train_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(__import__("random").randint(20000, 39999)), worker, str(tmp_path)],
                       capture_output=True, text=True, env=env, timeout=600)
    notes = "".join(open(os.path.join(str(tmp_path), f)).read()[-1500:] for f in sorted(os.listdir(str(tmp_path))) if f.endswith(".err"))
    assert r.returncode == 0, notes + r.stdout[-1000:] + r.stderr[-1000:]
    assert "DIST_TRAIN_OK" in r.stdout


def test_checkpoint_and_resume_through_the_file(spg, tmp_path):
    """Train, save with the optimiser sections, load: the loaded network carries the same weights, Adam moments and
    step counter, and training it further gives bit for bit what training the original further gives."""
    rng = np.random.default_rng(7)
    n = 512
    x = rng.random((n, 64), dtype=np.float32)
    t = np.zeros((n, 5), np.float32)
    t[np.arange(n), rng.integers(0, 5, n)] = 1.0
    net = spg.Network.build([64, 48, 5], [spg.abi.ACT_RELU, spg.abi.ACT_SOFTMAX], spg.abi.WEIGHT_INITIALIZATION_HE, seed=11)
    kw = dict(batch_size=n, strategy=spg.abi.STRATEGY_FULL_BATCH, learning_rate=1e-2)
    net.train(x, t, epochs=5, **kw)
    path = str(tmp_path / "ckpt.nn")
    net.save(path, spg.abi.PRECISION_FLOAT32, with_optimizer=True)
    back = spg.Network.load(path)
    assert back.c.time_step == net.c.time_step == 5
    assert np.array_equal(back.weights, net.weights) and np.array_equal(back.biases, net.biases)
    tw = int(net.c.total_weights)
    for name in ("opt_m_weights", "opt_v_weights"):
        a = np.ctypeslib.as_array(getattr(net.c, name), (tw,))
        b = np.ctypeslib.as_array(getattr(back.c, name), (tw,))
        assert np.array_equal(a, b) and np.any(a != 0), name
    net.train(x, t, epochs=4, **kw)
    back.train(x, t, epochs=4, **kw)
    assert back.c.time_step == net.c.time_step == 9
    assert np.array_equal(back.weights, net.weights) and np.array_equal(back.biases, net.biases)
    net.free()
    back.free()


@pytest.mark.parametrize("rows,fi,fo", [(256, 784, 512), (256, 1000, 10), (37, 53, 29), (37, 53, 7), (1024, 1031, 640), (300, 20, 1000),
                                        (37, 64, 48), (256, 512, 1000)])
def test_training_products_match_float64(spg, rows, fi, fo):
    """The three products of a training step and the one-launch weight+bias gradient against float64 numpy, on shapes
    that take each kernel (64x64 SIMT tiles; 32x32 tensor-core tiles with four or eight k-slices; the narrow-layer
    forward kernel, aligned and not) with whole and ragged tiles, aligned and unaligned operands."""
    import torch
    lib = spg.lib()
    vp, u32, f32 = C.c_void_p, C.c_uint32, C.c_float
    lib.spgk_train_gemm.argtypes = [C.c_int, vp, u32, vp, u32, vp, u32, u32, u32, u32, f32, vp, vp, u32, C.c_int, vp]
    lib.spgk_train_grad.argtypes = [vp, u32, vp, u32, vp, u32, vp, u32, u32, u32, f32, vp]
    rng = np.random.default_rng(rows * 7 + fi)
    x = rng.standard_normal((rows, fi)).astype(np.float32)
    w = (rng.standard_normal((fo, fi)) / np.sqrt(fi)).astype(np.float32)
    b = rng.standard_normal(fo).astype(np.float32)
    d = rng.standard_normal((rows, fo)).astype(np.float32)
    dx, dw, db, dd = (torch.from_numpy(a).cuda() for a in (x, w, b, d))
    tol = lambda ref: 2e-6 * max(1.0, float(np.abs(ref).max())) * np.sqrt(max(rows, fi, fo))
    # forward with ReLU
    y = torch.empty(rows, fo, device="cuda")
    assert lib.spgk_train_gemm(0, dx.data_ptr(), fi, dw.data_ptr(), fi, y.data_ptr(), fo, rows, fo, fi, 1.0, db.data_ptr(), None, 0,
                               spg.abi.ACT_RELU, None) == 0
    ref = np.maximum(x.astype(np.float64) @ w.astype(np.float64).T + b, 0.0)
    assert np.abs(y.cpu().numpy() - ref).max() <= tol(ref)
    # delta back through the layer, times the ReLU derivative of the layer input's activation
    act_in = np.maximum(x, 0.0)
    da = torch.from_numpy(act_in).cuda()
    dprev = torch.empty(rows, fi, device="cuda")
    assert lib.spgk_train_gemm(1, dd.data_ptr(), fo, dw.data_ptr(), fi, dprev.data_ptr(), fi, rows, fi, fo, 1.0, None, da.data_ptr(), fi,
                               spg.abi.ACT_RELU, None) == 0
    ref = (d.astype(np.float64) @ w.astype(np.float64)) * (act_in > 0)
    assert np.abs(dprev.cpu().numpy() - ref).max() <= tol(ref)
    # gradients: the product alone, then product + column sums in one launch; the product must not change
    gs = 1.0 / rows
    gw0 = torch.empty(fo, fi, device="cuda")
    gw1 = torch.empty(fo, fi, device="cuda")
    gb = torch.full((fo,), 7.0, device="cuda")
    assert lib.spgk_train_gemm(2, dd.data_ptr(), fo, dx.data_ptr(), fi, gw0.data_ptr(), fi, fo, fi, rows, gs, None, None, 0, 0, None) == 0
    assert lib.spgk_train_grad(dd.data_ptr(), fo, dx.data_ptr(), fi, gw1.data_ptr(), fi, gb.data_ptr(), fo, fi, rows, gs, None) == 0
    ref = gs * (d.astype(np.float64).T @ x.astype(np.float64))
    assert np.abs(gw0.cpu().numpy() - ref).max() <= tol(ref)
    assert torch.equal(gw0, gw1)
    refb = gs * d.astype(np.float64).sum(axis=0)
    assert np.abs(gb.cpu().numpy() - refb).max() <= tol(refb)


def test_a_c_program_written_against_the_public_header_trains_xor(spg, tmp_path):
    """tests/c/xor_program.c (MSE loss, FOO52 + sigmoid, AdamW with weight decay, callback, save / load / forward through the
    reference's macros) compiled with gcc against include/ and linked to the library: four OK lines, exit status 0."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "xor_program")
    libdir = os.path.dirname(spg.LIB_PATH)
    r = subprocess.run(["gcc", "-std=c2x", "-O1", "-I", os.path.join(root, "include"), os.path.join(root, "tests", "c", "xor_program.c"),
                        "-o", exe, "-L", libdir, "-lspingalett", "-lm", "-Wl,-rpath," + libdir], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    run = subprocess.run([exe], capture_output=True, text=True, cwd=str(tmp_path), timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert run.stdout.count("OK in=") == 4 and "passed 4/4, reloaded 4/4" in run.stdout
