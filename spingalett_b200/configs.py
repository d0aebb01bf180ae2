"""Builders for the benchmark configurations used by the benchmark and the GPU parity tests: seeded weights, written to a .nn file in the wanted precision by
the library's own save_spingalett (byte-identical to the reference writer, see
test_host_abi.py), and seeded synthetic inputs.  Nothing here needs the
reference checkout."""
import os

import numpy as np

from . import abi

A_TOPO, A_ACTS = [784, 512, 1000, 10], [abi.ACT_RELU, abi.ACT_RELU, abi.ACT_SOFTMAX]
W_TOPO = [4096, 8192, 8192, 8192, 8192, 4096, 1000]
W_ACTS = [abi.ACT_LEAKY_RELU] * 4 + [abi.ACT_TANH, abi.ACT_SOFTMAX]
L_TOPO, L_ACTS = [8192, 16384, 16384, 8192, 1000], [abi.ACT_FOO52] * 3 + [abi.ACT_SOFTMAX]


def fill_normal(net, topo, gain, seed):
    """He (gain 2) / "Xavier" (gain 1) style N(0,1)*sqrt(gain/fan_in) weights, zero biases,
    drawn with numpy (fast enough for the half-billion-weight configurations)."""
    rng = np.random.default_rng(seed)
    w = net.weights
    pos = 0
    for l in range(len(topo) - 1):
        cnt = topo[l] * topo[l + 1]
        w[pos:pos + cnt] = rng.standard_normal(cnt, dtype=np.float32) * np.float32(np.sqrt(gain / topo[l]))
        pos += cnt
    net.biases[:] = 0.0


def make_net_file(spg, path, topo, acts, precision, *, gain=2.0, seed=1234, reference_rng=False):
    """Writes `path` (a .nn file of the given precision) unless it exists already."""
    if os.path.exists(path):
        return path
    if reference_rng:
        init = abi.WEIGHT_INITIALIZATION_HE if gain == 2.0 else abi.WEIGHT_INITIALIZATION_XAVIER
        net = spg.Network.build(topo, acts, init, seed=seed)
    else:
        net = spg.Network.build(topo, acts, abi.WEIGHT_INITIALIZATION_NONE)
        fill_normal(net, topo, gain, seed)
    net.save(path, precision)
    net.free()
    return path


def uniform_inputs(n, width, seed=99):
    return np.random.default_rng(seed).random((n, width), dtype=np.float32)


def normal_inputs(n, width, seed=99):
    return np.random.default_rng(seed).standard_normal((n, width), dtype=np.float32)


def parity(got, want):
    """(argmax agreement fraction, max abs error) between two [N][C] outputs."""
    agree = float(np.mean(np.argmax(got, 1) == np.argmax(want, 1)))
    return agree, float(np.abs(got - want).max())


def tolerance(precision):
    """Max-abs softmax error allowed: 2e-3 for float files, 5e-3 for integer files."""
    return 2e-3 if precision <= abi.PRECISION_BFLOAT16 else 5e-3
