"""Regenerates the golden fixtures in this directory by RUNNING THE REFERENCE.

The reference (pka-human/Spingalett) ships no test vectors, so the known-answer
data that pins the oracle and the CUDA library is produced here by the
reference's own code, compiled unmodified into oracle/_ref (see
oracle/Makefile).  Needs the reference checkout; the committed outputs are what
the test-suite reads, on machines that do not have it.

    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import Reference, build_reference  # noqa: E402
from spingalett_b200 import abi  # noqa: E402

PRECS = ["fp32", "fp16", "bf16", "int8", "int4", "int2"]


# (name, strategy, optimizer, loss, output activation, weight decay, max_grad_norm, epochs, batch)
TRAIN_CASES = [
    ("sgd_decay", abi.STRATEGY_FULL_BATCH, abi.OPTIMIZER_SGD, abi.LOSS_CROSS_ENTROPY, abi.ACT_SOFTMAX, 1e-3, 0.0, 6, 0),
    ("momentum_decay", abi.STRATEGY_FULL_BATCH, abi.OPTIMIZER_MOMENTUM, abi.LOSS_CROSS_ENTROPY, abi.ACT_SOFTMAX, 1e-3, 0.0, 6, 0),
    ("rmsprop_decay", abi.STRATEGY_FULL_BATCH, abi.OPTIMIZER_RMSPROP, abi.LOSS_CROSS_ENTROPY, abi.ACT_SOFTMAX, 1e-3, 0.0, 6, 0),
    ("adam_decay", abi.STRATEGY_FULL_BATCH, abi.OPTIMIZER_ADAM, abi.LOSS_CROSS_ENTROPY, abi.ACT_SOFTMAX, 1e-3, 0.0, 6, 0),
    ("adamw_decay", abi.STRATEGY_FULL_BATCH, abi.OPTIMIZER_ADAMW, abi.LOSS_CROSS_ENTROPY, abi.ACT_SOFTMAX, 1e-2, 0.0, 6, 0),
    ("sgd_clip", abi.STRATEGY_FULL_BATCH, abi.OPTIMIZER_SGD, abi.LOSS_CROSS_ENTROPY, abi.ACT_SOFTMAX, 0.0, 0.05, 6, 0),
    ("mse_sigmoid_adamw", abi.STRATEGY_FULL_BATCH, abi.OPTIMIZER_ADAMW, abi.LOSS_MSE, abi.ACT_SIGMOID, 1e-4, 0.0, 6, 0),
    ("mse_softmax_sgd", abi.STRATEGY_FULL_BATCH, abi.OPTIMIZER_SGD, abi.LOSS_MSE, abi.ACT_SOFTMAX, 0.0, 0.0, 6, 0),
    ("ce_tanh_out_sgd", abi.STRATEGY_FULL_BATCH, abi.OPTIMIZER_SGD, abi.LOSS_CROSS_ENTROPY, abi.ACT_TANH, 0.0, 0.0, 4, 0),
    ("sample_momentum", abi.STRATEGY_SAMPLE, abi.OPTIMIZER_MOMENTUM, abi.LOSS_MSE, abi.ACT_SIGMOID, 1e-3, 0.0, 2, 0),
]


def make_train_surface(R, L, rng):
    """Final weights, biases and reported loss of the reference's train() for every update rule and output-delta form,
    each starting from tests/golden/train.fp32.nn (output activation and loss overridden in the public struct) on the
    batch stored in train.npz."""
    d = np.load(os.path.join(HERE, "train.npz"))
    x, t = np.ascontiguousarray(d["x"]), np.ascontiguousarray(d["t"])
    out = {}
    losses = {}

    def on_epoch(net, epoch, err):
        on_epoch.last = float(err)
        return False
    cb = abi.TrainCallback(on_epoch)
    for name, strat, opt, loss, out_act, decay, clip, epochs, batch in TRAIN_CASES:
        net = R.load(os.path.join(HERE, "train.fp32.nn"))
        c = net.contents
        c.act_func[c.layers - 2] = out_act
        c.loss_func = loss
        L.spingalett_set_compute_mode(abi.COMPUTE_OPENBLAS)
        a = abi.TrainArgs()
        a.net = net
        a.training_strategy, a.optimizer_type = strat, opt
        a.inputs, a.targets = x.ctypes.data, t.ctypes.data
        a.sample_count, a.batch_size, a.epochs = x.shape[0], batch, epochs
        a.learning_rate, a.weight_decay, a.max_grad_norm = 0.01, decay, clip
        a.callback, a.callback_interval = cb, 1
        L.train_struct_arguments(a)
        assert L.spingalett_last_error_code() == 0, name
        out[name + ".w"] = R.weights(net).copy()
        out[name + ".b"] = R.biases(net).copy()
        losses[name] = on_epoch.last
        R.free(net)
    L.spingalett_set_compute_mode(abi.COMPUTE_SINGLE_THREADED)
    np.savez(os.path.join(HERE, "train_surface.npz"), **out, **{k + ".loss": np.float32(v) for k, v in losses.items()})


def main():
    assert build_reference() is not None, "reference checkout not found"
    R = Reference
    L = R.lib()
    L.spingalett_set_compute_mode(abi.COMPUTE_SINGLE_THREADED)
    rng = np.random.default_rng(20240607)
    meta = {"generator": "tests/golden/make_golden.py", "reference_blas": bool(L.refh_has_blas()), "nets": {}}

    # -- generator stream: raw words, uniforms and normals after seed 1234 ------
    L.refh_rng_seed(1234)
    words = np.array([L.refh_rng_next() for _ in range(32)], np.uint32)
    L.refh_rng_seed(1234)
    normals = np.array([L.refh_normal() for _ in range(32)], np.float32)
    L.refh_rng_seed(1234)
    uniforms = np.array([L.refh_uniform() for _ in range(32)], np.float32)
    np.savez(os.path.join(HERE, "rng_seed1234.npz"), words=words, normals=normals, uniforms=uniforms)

    # -- activations on edge values (exported activate()/derivative()) ----------
    xs = np.array([0.0, -0.0, 1.0, -1.0, 1e-8, -1e-8, 1.0000001, 0.99999994, 0.5, -0.5, 3.75, -3.75, 20.0, -20.0,
                   88.0, -88.0, 100.0, -100.0, 1e30, -1e30, np.inf, -np.inf], np.float32)
    act_tab = np.zeros((abi.ACT_COUNT, xs.size), np.float32)
    der_tab = np.zeros((abi.ACT_COUNT, xs.size), np.float32)
    for a in range(abi.ACT_COUNT):
        for i, v in enumerate(xs):
            act_tab[a, i] = L.activate(float(v), a)
            der_tab[a, i] = L.derivative(float(v), a)
    np.savez(os.path.join(HERE, "activations.npz"), x=xs, activate=act_tab, derivative=der_tab)

    # -- softmax rows (apply_softmax) -------------------------------------------
    rows = [rng.normal(0, 3, 10), rng.normal(0, 1, 1000), np.full(7, -1e30), np.array([1e30, -1e30, 0.0]),
            np.array([5.0]), np.array([88.0, 89.0, -90.0, 0.0]), np.zeros(33)]
    sm_in, sm_out = [], []
    for r in rows:
        r = np.ascontiguousarray(r, np.float32)
        o = r.copy()
        L.refh_softmax(o.ctypes.data_as(abi.f32p), o.size)
        sm_in.append(r)
        sm_out.append(o)
    np.savez(os.path.join(HERE, "softmax.npz"), **{f"in{i}": a for i, a in enumerate(sm_in)},
             **{f"out{i}": a for i, a in enumerate(sm_out)})

    # -- small nets saved by the reference at every precision -------------------
    specs = {
        # name: (topology, activations, init, seed)
        "small": ([20, 33, 17, 10], [abi.ACT_RELU, abi.ACT_FOO52, abi.ACT_SOFTMAX], abi.WEIGHT_INITIALIZATION_HE, 7),
        # odd widths: 4- and 2-bit rows start in the middle of a byte
        "odd": ([15, 9, 7, 5], [abi.ACT_TANH, abi.ACT_LEAKY_RELU, abi.ACT_SIGMOID], abi.WEIGHT_INITIALIZATION_XAVIER, 11),
        # every 8-aligned width, no softmax, linear output
        "wide8": ([64, 136, 72, 24], [abi.ACT_LEAKY_RELU, abi.ACT_SIGMOID, abi.ACT_NONE], abi.WEIGHT_INITIALIZATION_RANDOM, 13),
    }
    for name, (topo, acts, init, seed) in specs.items():
        net = R.build_net(topo, acts, init, seed=seed)
        # non-zero biases so the bias codec is exercised too
        b = R.biases(net)
        b[:] = rng.normal(0, 0.1, b.size).astype(np.float32)
        x = rng.random((16, topo[0]), dtype=np.float32) * 2 - 0.5
        np.save(os.path.join(HERE, f"{name}.inputs.npy"), x)
        meta["nets"][name] = {"topology": topo, "acts": acts, "init": init, "seed": seed}
        for p, pname in enumerate(PRECS):
            path = os.path.join(HERE, f"{name}.{pname}.nn")
            R.save(net, path, p)
            loaded = R.load(path)
            np.save(os.path.join(HERE, f"{name}.{pname}.weights.npy"),
                    np.concatenate([R.weights(loaded), R.biases(loaded)]).copy())
            y = np.stack([R.forward(loaded, xi) for xi in x])
            np.save(os.path.join(HERE, f"{name}.{pname}.outputs.npy"), y)
            R.free(loaded)
        R.free(net)

    # -- a file that carries optimizer state and a time step --------------------
    net = R.build_net([6, 5, 4], [abi.ACT_RELU, abi.ACT_SOFTMAX], abi.WEIGHT_INITIALIZATION_HE, seed=3)
    c = net.contents
    for arr, n in [(c.opt_m_weights, c.total_weights), (c.opt_v_weights, c.total_weights),
                   (c.opt_m_biases, c.total_biases), (c.opt_v_biases, c.total_biases)]:
        np.ctypeslib.as_array(arr, shape=(n,))[:] = rng.normal(0, 0.01, n).astype(np.float32)
    c.time_step = 42
    for pname in ("fp32", "int8"):
        path = os.path.join(HERE, f"withopt.{pname}.nn")
        R.save(net, path, PRECS.index(pname), with_optimizer=True)
        loaded = R.load(path)
        lc = loaded.contents
        np.savez(os.path.join(HERE, f"withopt.{pname}.state.npz"),
                 weights=R.weights(loaded).copy(), biases=R.biases(loaded).copy(),
                 m_w=np.ctypeslib.as_array(lc.opt_m_weights, shape=(lc.total_weights,)).copy(),
                 v_w=np.ctypeslib.as_array(lc.opt_v_weights, shape=(lc.total_weights,)).copy(),
                 m_b=np.ctypeslib.as_array(lc.opt_m_biases, shape=(lc.total_biases,)).copy(),
                 v_b=np.ctypeslib.as_array(lc.opt_v_biases, shape=(lc.total_biases,)).copy(),
                 time_step=np.uint64(lc.time_step))
        R.free(loaded)
    R.free(net)

    # -- one training batch: gradients and ten Adam steps ----------------------
    if L.refh_has_blas():
        topo, acts = [12, 16, 8, 5], [abi.ACT_RELU, abi.ACT_TANH, abi.ACT_SOFTMAX]
        net = R.build_net(topo, acts, abi.WEIGHT_INITIALIZATION_HE, loss=abi.LOSS_CROSS_ENTROPY, seed=21)
        path = os.path.join(HERE, "train.fp32.nn")
        R.save(net, path, 0)
        N = 24
        x = rng.random((N, topo[0]), dtype=np.float32)
        t = np.zeros((N, topo[-1]), np.float32)
        t[np.arange(N), rng.integers(0, topo[-1], N)] = 1.0
        L.spingalett_set_compute_mode(abi.COMPUTE_OPENBLAS)
        assert L.refh_batch_gradients(net, x.ctypes.data_as(abi.f32p), t.ctypes.data_as(abi.f32p), N, 1.0 / N) == 0
        c = net.contents
        g = np.concatenate([np.ctypeslib.as_array(c.grad_weights, shape=(c.total_weights,)),
                            np.ctypeslib.as_array(c.grad_biases, shape=(c.total_biases,))]).copy()
        # Adam on a small vector, steps 1..10, factors formed as train() forms them
        w = rng.normal(0, 0.1, 37).astype(np.float32)
        w0 = w.copy()
        m = np.zeros_like(w)
        v = np.zeros_like(w)
        b1p = b2p = np.float32(1.0)
        b1, b2, lr, eps = np.float32(0.9), np.float32(0.999), np.float32(1e-3), np.float32(1e-8)
        steps_w, grads = [], []
        for _ in range(10):
            gs = rng.normal(0, 0.05, w.size).astype(np.float32)
            b1p = np.float32(b1p * b1)
            b2p = np.float32(b2p * b2)
            mf = np.float32(1.0) / (np.float32(1.0) - b1p)
            vf = np.float32(1.0) / (np.float32(1.0) - b2p)
            L.refh_adam(w.ctypes.data_as(abi.f32p), m.ctypes.data_as(abi.f32p), v.ctypes.data_as(abi.f32p),
                        gs.ctypes.data_as(abi.f32p), w.size, lr, b1, b2, mf, vf, eps)
            steps_w.append(w.copy())
            grads.append(gs)
        np.savez(os.path.join(HERE, "train.npz"), x=x, t=t, grads=g, adam_w=np.stack(steps_w), adam_g=np.stack(grads),
                 adam_m=m, adam_v=v, adam_w0=w0)
        L.spingalett_set_compute_mode(abi.COMPUTE_SINGLE_THREADED)
        R.free(net)

    # -- the rest of the train() surface: one short run of the reference's own train() per update rule / loss ----------
    if L.refh_has_blas():
        make_train_surface(R, L, rng)

    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(meta, f, indent=1)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
