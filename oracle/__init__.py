"""Test-only checkers for the CUDA library.

`Oracle`    -- ctypes face of libspg_oracle.so, the plain-C restatement of the
               reference's forward path (spg_oracle.c).
`Reference` -- ctypes face of _ref/libspingalett_ref.so, the UNMODIFIED
               reference compiled from its own sources plus ref_harness.c.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import
this package; the product (spingalett_b200) never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

from spingalett_b200 import abi

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libspg_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libspingalett_ref.so")


def build_oracle():
    subprocess.run(["make", "-C", HERE, "oracle"], check=True, capture_output=True)
    return ORACLE_SO


def reference_root():
    """Where the reference checkout is looked for: $SPINGALETT_REFERENCE, else a directory named reference beside this
    repository."""
    return os.environ.get("SPINGALETT_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build_reference(ref_root=None):
    """Compile the reference where it lies; returns None when no checkout exists."""
    ref_root = ref_root or reference_root()
    if not os.path.isdir(os.path.join(ref_root, "Src")):
        return REF_SO if os.path.exists(REF_SO) else None
    subprocess.run(["make", "-C", HERE, "ref", f"REF={ref_root}"], check=True, capture_output=True)
    return REF_SO


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


_fp = C.POINTER(C.c_float)


def _p(a):
    return a.ctypes.data_as(_fp)


class Oracle:
    _lib = None

    @classmethod
    def lib(cls):
        if cls._lib is None:
            if not os.path.exists(ORACLE_SO):
                build_oracle()
            l = C.CDLL(ORACLE_SO)
            l.spgo_parse.restype = C.c_void_p
            l.spgo_parse.argtypes = [C.c_char_p, C.c_uint64]
            l.spgo_from_arrays.restype = C.c_void_p
            l.spgo_from_arrays.argtypes = [C.c_uint32, C.c_void_p, C.c_void_p, _fp, _fp]
            l.spgo_free.argtypes = [C.c_void_p]
            for name, rt in [("spgo_layers", C.c_uint32), ("spgo_topology", C.POINTER(C.c_uint32)),
                             ("spgo_acts", C.POINTER(C.c_uint8)), ("spgo_weights", _fp), ("spgo_biases", _fp),
                             ("spgo_total_weights", C.c_uint64), ("spgo_total_biases", C.c_uint64),
                             ("spgo_precision", C.c_int), ("spgo_truncated", C.c_int),
                             ("spgo_has_optimizer", C.c_int), ("spgo_time_step", C.c_uint64), ("spgo_loss", C.c_int)]:
                getattr(l, name).restype = rt
                getattr(l, name).argtypes = [C.c_void_p]
            l.spgo_forward.argtypes = [C.c_void_p, _fp, _fp]
            l.spgo_forward_batch.argtypes = [C.c_void_p, _fp, C.c_uint64, _fp]
            l.spgo_forward_batch_acts.argtypes = [C.c_void_p, _fp, C.c_uint64, _fp]
            l.spgo_batch_gradients.argtypes = [C.c_void_p, _fp, _fp, C.c_uint32, C.c_float, _fp]
            l.spgo_adam.argtypes = [_fp, _fp, _fp, _fp, C.c_uint64] + [C.c_float] * 6
            l.spgo_array_bytes.restype = C.c_uint64
            l.spgo_array_bytes.argtypes = [C.c_uint64, C.c_int]
            l.spgo_decode_array.argtypes = [C.c_void_p, C.c_uint64, C.c_int, _fp]
            l.spgo_encode_array.restype = C.c_uint64
            l.spgo_encode_array.argtypes = [_fp, C.c_uint64, C.c_int, C.c_void_p]
            l.spgo_activate.restype = C.c_float
            l.spgo_activate.argtypes = [C.c_float, C.c_int]
            l.spgo_derivative.restype = C.c_float
            l.spgo_derivative.argtypes = [C.c_float, C.c_int]
            l.spgo_softmax.argtypes = [_fp, C.c_uint32]
            l.spgo_dot.restype = C.c_float
            l.spgo_dot.argtypes = [_fp, _fp, C.c_uint64]
            l.spgo_cross_entropy.restype = C.c_float
            l.spgo_cross_entropy.argtypes = [_fp, _fp, C.c_uint32]
            l.spgo_threads.restype = C.c_int
            cls._lib = l
        return cls._lib

    # -- codecs --------------------------------------------------------------
    @classmethod
    def encode(cls, values, precision):
        v = _f32(values).ravel()
        n = cls.lib().spgo_array_bytes(v.size, precision)
        buf = np.zeros(n, np.uint8)
        cls.lib().spgo_encode_array(_p(v), v.size, precision, buf.ctypes.data)
        return buf

    @classmethod
    def decode(cls, raw, count, precision):
        raw = np.ascontiguousarray(raw, np.uint8)
        out = np.empty(count, np.float32)
        cls.lib().spgo_decode_array(raw.ctypes.data, count, precision, _p(out))
        return out

    @classmethod
    def activate(cls, x, act):
        return np.array([cls.lib().spgo_activate(float(v), act) for v in np.ravel(x)], np.float32)

    @classmethod
    def softmax(cls, row):
        r = _f32(row).copy()
        cls.lib().spgo_softmax(_p(r), r.size)
        return r

    @classmethod
    def threads(cls):
        return cls.lib().spgo_threads()


class OracleNet:
    """A network held by the oracle: parsed from .nn bytes or built from arrays."""

    def __init__(self, handle):
        if not handle:
            raise ValueError("oracle rejected the network image")
        self.h = handle
        l = Oracle.lib()
        self.layers = l.spgo_layers(self.h)
        self.topology = [l.spgo_topology(self.h)[i] for i in range(self.layers)]
        self.acts = [l.spgo_acts(self.h)[i] for i in range(self.layers - 1)]
        self.precision = l.spgo_precision(self.h)
        self.truncated = bool(l.spgo_truncated(self.h))
        self.has_optimizer = bool(l.spgo_has_optimizer(self.h))
        self.time_step = l.spgo_time_step(self.h)
        self.loss = l.spgo_loss(self.h)

    @classmethod
    def from_file(cls, path):
        with open(path, "rb") as f:
            data = f.read()
        return cls.from_bytes(data)

    @classmethod
    def from_bytes(cls, data):
        h = Oracle.lib().spgo_parse(data, len(data))
        if not h:
            return None
        return cls(h)

    @classmethod
    def from_arrays(cls, topology, acts, weights, biases):
        t = np.asarray(topology, np.uint32)
        a = np.asarray(acts, np.uint8)
        w, b = _f32(weights), _f32(biases)
        return cls(Oracle.lib().spgo_from_arrays(len(topology), t.ctypes.data, a.ctypes.data, _p(w), _p(b)))

    @property
    def weights(self):
        n = Oracle.lib().spgo_total_weights(self.h)
        return np.ctypeslib.as_array(Oracle.lib().spgo_weights(self.h), shape=(n,))

    @property
    def biases(self):
        n = Oracle.lib().spgo_total_biases(self.h)
        return np.ctypeslib.as_array(Oracle.lib().spgo_biases(self.h), shape=(n,))

    def forward(self, x):
        x = _f32(x)
        out = np.empty(self.topology[-1], np.float32)
        Oracle.lib().spgo_forward(self.h, _p(x), _p(out))
        return out

    def forward_batch(self, x):
        x = _f32(x)
        out = np.empty((x.shape[0], self.topology[-1]), np.float32)
        Oracle.lib().spgo_forward_batch(self.h, _p(x), x.shape[0], _p(out))
        return out

    def gradients(self, x, targets, scale):
        x, t = _f32(x), _f32(targets)
        g = np.empty(len(self.weights) + len(self.biases), np.float32)
        Oracle.lib().spgo_batch_gradients(self.h, _p(x), _p(t), x.shape[0], scale, _p(g))
        return g

    def __del__(self):
        try:
            Oracle.lib().spgo_free(self.h)
        except Exception:
            pass


class Reference:
    """The unmodified reference library (only where oracle/_ref was built)."""
    _lib = None

    @classmethod
    def available(cls):
        return os.path.exists(REF_SO)

    @classmethod
    def lib(cls):
        if cls._lib is None:
            l = C.CDLL(REF_SO)
            abi.bind_reference_abi(l)
            l.refh_rng_seed.argtypes = [C.c_uint64]
            l.refh_has_blas.restype = C.c_int
            l.refh_blas_threads.argtypes = [C.c_int]
            l.refh_batch_forward.argtypes = [abi.NetP, _fp, C.c_uint32, _fp]
            l.refh_batch_forward.restype = C.c_int
            l.refh_ws_create.argtypes = [abi.NetP, C.c_uint32]
            l.refh_ws_create.restype = C.c_void_p
            l.refh_ws_free.argtypes = [C.c_void_p]
            l.refh_ws_forward.argtypes = [abi.NetP, C.c_void_p, _fp, C.c_uint32]
            l.refh_ws_forward.restype = _fp
            l.refh_batch_gradients.argtypes = [abi.NetP, _fp, _fp, C.c_uint32, C.c_float]
            l.refh_batch_gradients.restype = C.c_int
            l.refh_adam.argtypes = [_fp, _fp, _fp, _fp, C.c_uint64] + [C.c_float] * 6
            l.refh_dot.restype = C.c_float
            l.refh_dot.argtypes = [_fp, _fp, C.c_uint64]
            l.refh_softmax.argtypes = [_fp, C.c_uint32]
            l.refh_activation_bulk.argtypes = [_fp, C.c_uint64, C.c_int]
            l.refh_normal.restype = C.c_float
            l.refh_uniform.restype = C.c_float
            l.refh_rng_next.restype = C.c_uint32
            l.refh_sizeof_net.restype = C.c_size_t
            l.refh_sizeof_trainargs.restype = C.c_size_t
            l.spingalett_set_verbose(False)
            cls._lib = l
        return cls._lib

    @classmethod
    def build_net(cls, topology, acts, init, loss=abi.LOSS_CROSS_ENTROPY, seed=None):
        l = cls.lib()
        if seed is not None:
            l.refh_rng_seed(seed)
        net = l.new_spingalett_struct_arguments(abi.NeuralNetworkArgs(loss))
        l.layer_struct_arguments(abi.LayerArgs(net, topology[0], 0, 0))
        for w, a in zip(topology[1:], acts):
            l.layer_struct_arguments(abi.LayerArgs(net, w, a, init))
        return net

    @classmethod
    def weights(cls, net):
        return np.ctypeslib.as_array(net.contents.weights, shape=(net.contents.total_weights,))

    @classmethod
    def biases(cls, net):
        return np.ctypeslib.as_array(net.contents.biases, shape=(net.contents.total_biases,))

    @classmethod
    def save(cls, net, path, precision, with_optimizer=False):
        cls.lib().save_spingalett_struct_arguments(abi.SaveArgs(net, os.fsencode(path), not with_optimizer, precision))

    @classmethod
    def load(cls, path):
        cls.lib().spingalett_clear_error()
        return cls.lib().load_spingalett(os.fsencode(path))

    @classmethod
    def forward(cls, net, x):
        x = _f32(x)
        n_out = net.contents.topology[net.contents.layers - 1]
        o = cls.lib().forward_struct_arguments(abi.ForwardArgs(net, _p(x)))
        return np.ctypeslib.as_array(o, shape=(n_out,)).copy()

    @classmethod
    def forward_batch(cls, net, x):
        x = _f32(x)
        n_out = net.contents.topology[net.contents.layers - 1]
        out = np.empty((x.shape[0], n_out), np.float32)
        if cls.lib().refh_has_blas():
            cls.lib().spingalett_set_compute_mode(abi.COMPUTE_OPENBLAS)
        rc = cls.lib().refh_batch_forward(net, _p(x), x.shape[0], _p(out))
        assert rc == 0
        return out

    @classmethod
    def free(cls, net):
        cls.lib().free_network(net)
