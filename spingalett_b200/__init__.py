"""spingalett_b200 -- Python face of the B200-native Spingalett library.

The product is the C-ABI shared library `lib/libspingalett.so` (C23 host code +
hand-written sm_100a CUDA kernels).  This module only loads it and mirrors the
reference's operator interface (new_spingalett / layer / forward / train /
save_spingalett / load_spingalett) one to one, so tests read like programs
written against the reference.  There is no Python or CPU compute path: if the
library has not been built, importing `lib()` raises.
"""
import ctypes as C
import os

import numpy as np

from . import abi
from .abi import *  # noqa: F401,F403  (enumerators)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libspingalett.so")
_lib = None


def lib():
    """The loaded libspingalett.so (raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libspingalett.so is not built (run `python -m spingalett_b200.build`); "
                "this package has no fallback implementation")
        handle = C.CDLL(LIB_PATH)
        abi.bind_reference_abi(handle)
        abi.bind_extensions(handle)
        _lib = handle
    return _lib


class SpingalettError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"spingalett error {code}: {message}")
        self.code = code


def _check():
    l = lib()
    code = l.spingalett_last_error_code()
    if code != abi.OK:
        msg = l.spingalett_last_error_message().decode(errors="replace")
        l.spingalett_clear_error()
        raise SpingalettError(code, msg)


def _as_f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Network:
    """Owns one NeuralNetwork* of the C library."""

    def __init__(self, handle):
        if not handle:
            _check()
            raise SpingalettError(-1, "NULL network")
        self._h = handle

    # -- construction (reference: new_spingalett + layer, Network.c:34-200) --
    @classmethod
    def new(cls, loss=abi.LOSS_MSE):
        lib().spingalett_clear_error()
        return cls(lib().new_spingalett_struct_arguments(abi.NeuralNetworkArgs(loss)))

    def layer(self, neurons, act=abi.ACT_SIGMOID, init=abi.WEIGHT_INITIALIZATION_RANDOM):
        lib().layer_struct_arguments(abi.LayerArgs(self._h, neurons, act, init))
        _check()
        return self

    @classmethod
    def build(cls, topology, acts, init=abi.WEIGHT_INITIALIZATION_HE, loss=abi.LOSS_CROSS_ENTROPY, seed=None):
        if seed is not None:
            lib().spingalett_seed(seed)
        net = cls.new(loss)
        net.layer(topology[0])
        for width, act in zip(topology[1:], acts):
            net.layer(width, act, init)
        return net

    @classmethod
    def load(cls, path):
        lib().spingalett_clear_error()
        h = lib().load_spingalett(os.fsencode(path))
        return cls(h)

    def save(self, path, precision=abi.PRECISION_FLOAT32, with_optimizer=False):
        lib().save_spingalett_struct_arguments(abi.SaveArgs(self._h, os.fsencode(path), not with_optimizer, precision))
        _check()

    def free(self):
        if self._h:
            lib().free_network(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    # -- views of the public struct ---------------------------------------
    @property
    def c(self):
        return self._h.contents

    @property
    def topology(self):
        return [self.c.topology[i] for i in range(self.c.layers)]

    @property
    def acts(self):
        return [self.c.act_func[i] for i in range(self.c.layers - 1)]

    def _view(self, ptr, count):
        if not ptr or count == 0:
            return np.zeros(0, np.float32)
        return np.ctypeslib.as_array(ptr, shape=(count,))

    @property
    def weights(self):
        return self._view(self.c.weights, self.c.total_weights)

    @property
    def biases(self):
        return self._view(self.c.biases, self.c.total_biases)

    def sync_weights(self):
        if lib().spingalett_sync_weights(self._h) != 0:
            _check()

    def train(self, inputs, targets, *, epochs=1, batch_size=0, strategy=abi.STRATEGY_SMALL_BATCH,
              optimizer=abi.OPTIMIZER_ADAM, learning_rate=0.0, beta1=0.0, beta2=0.0, epsilon=0.0,
              report_interval=0, reset_optimizer=False, nan_check_interval=0, callback=None, callback_interval=0,
              weight_decay=0.0, momentum=0.0, max_grad_norm=0.0, autosave_mode=0, autosave_interval=0, autosave_path=None,
              autosave_precision=abi.PRECISION_FLOAT32, autosave_with_optimizer=True):
        """reference train(): MODE_ARRAY over host arrays [samples][in] / [samples][out]."""
        x, t = _as_f32(inputs), _as_f32(targets)
        args = abi.TrainArgs()
        args.net = self._h
        args.training_mode = abi.MODE_ARRAY if hasattr(abi, "MODE_ARRAY") else 0
        args.training_strategy = strategy
        args.optimizer_type = optimizer
        args.inputs = x.ctypes.data
        args.targets = t.ctypes.data
        args.sample_count = x.shape[0]
        args.batch_size = batch_size
        args.epochs = epochs
        args.learning_rate = learning_rate
        args.beta1, args.beta2, args.epsilon = beta1, beta2, epsilon
        args.weight_decay, args.momentum, args.max_grad_norm = weight_decay, momentum, max_grad_norm
        args.autosave_mode, args.autosave_interval = autosave_mode, autosave_interval
        args.autosave_path = os.fsencode(autosave_path) if autosave_path else None
        args.autosave_precision = autosave_precision
        args.autosave_do_not_save_optimizer = not autosave_with_optimizer
        args.report_interval = report_interval
        args.reset_optimizer = reset_optimizer
        args.nan_check_interval = nan_check_interval
        if callback is not None:
            args.callback = abi.TrainCallback(callback)
            args.callback_interval = callback_interval
        lib().train_struct_arguments(args)
        _check()

    def synchronize(self):
        if lib().spingalett_synchronize(self._h) != 0:
            _check()

    def profile(self, enable=True):
        lib().spingalett_profile(self._h, enable)

    def profile_read(self):
        """(summed device milliseconds of the timed layer kernels, how many kernels) since the last read"""
        ms, cnt = C.c_double(0), C.c_uint64(0)
        lib().spingalett_profile_read(self._h, C.byref(ms), C.byref(cnt))
        return ms.value, cnt.value

    def set_stream(self, stream_handle):
        lib().spingalett_set_stream(self._h, C.c_void_p(stream_handle))

    # -- compute (always on the GPU) ----------------------------------------
    def forward(self, x):
        """reference forward(): one sample, returns a copy of the output layer."""
        x = _as_f32(x)
        assert x.size == self.topology[0]
        out = lib().forward_struct_arguments(abi.ForwardArgs(self._h, x.ctypes.data_as(abi.f32p)))
        if not out:
            _check()
            raise SpingalettError(-1, "forward returned NULL")
        return np.ctypeslib.as_array(out, shape=(self.topology[-1],)).copy()

    def forward_batch(self, x, out=None):
        """Batched inference on host arrays; returns [N][out] float32."""
        x = _as_f32(x)
        n = x.shape[0]
        if out is None:
            out = np.empty((n, self.topology[-1]), np.float32)
        r = lib().forward_batch_struct_arguments(
            abi.ForwardBatchArgs(self._h, x.ctypes.data, n, out.ctypes.data))
        if not r:
            _check()
            raise SpingalettError(-1, "forward_batch returned NULL")
        return out

    def forward_batch_ptr(self, in_ptr, n, out_ptr):
        """Batched inference on raw host/device pointers (used by the benchmark)."""
        r = lib().forward_batch_struct_arguments(abi.ForwardBatchArgs(self._h, in_ptr, n, out_ptr))
        if not r:
            _check()
            raise SpingalettError(-1, "forward_batch returned NULL")
        return r


def shard_rows(rows, world, rank):
    """Contiguous share [lo, hi) of `rows` batch rows for `rank` of `world` (sizes differ by at most one)."""
    base, extra = divmod(rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def set_math_mode(mode):
    lib().spingalett_set_math_mode(mode)


def last_path():
    return lib().spingalett_last_path().decode()


def kernel_launches():
    return int(lib().spingalett_kernel_launches())
