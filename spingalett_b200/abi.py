"""ctypes mirror of the C ABI in include/spingalett_b200.h.

The record layouts and enumerator values are those of pka-human/Spingalett's
Include/Spingalett/Spingalett.h (:28-196), which is why the same definitions
also bind the reference library itself when a test loads it as the checker.
"""
import ctypes as C

# enumerators (Spingalett.h:38-47, :93-101, :49-53, :55-61, :69-83)
ACT_SIGMOID, ACT_RELU, ACT_TANH, ACT_LEAKY_RELU, ACT_FOO52, ACT_SOFTMAX, ACT_NONE, ACT_COUNT = range(8)
PRECISION_FLOAT32, PRECISION_FP16, PRECISION_BFLOAT16, PRECISION_INT8, PRECISION_INT4, PRECISION_INT2, PRECISION_COUNT = range(7)
LOSS_MSE, LOSS_CROSS_ENTROPY = 0, 1
WEIGHT_INITIALIZATION_RANDOM, WEIGHT_INITIALIZATION_XAVIER, WEIGHT_INITIALIZATION_HE, WEIGHT_INITIALIZATION_NONE = range(4)
STRATEGY_SAMPLE, STRATEGY_FULL_BATCH, STRATEGY_SMALL_BATCH = range(3)
OPTIMIZER_SGD, OPTIMIZER_MOMENTUM, OPTIMIZER_RMSPROP, OPTIMIZER_ADAM, OPTIMIZER_ADAMW = range(5)
COMPUTE_SINGLE_THREADED, COMPUTE_OPENMP, COMPUTE_OPENBLAS, COMPUTE_CUDA = range(4)
LOG_DEBUG, LOG_INFO, LOG_WARNING, LOG_ERROR, LOG_NONE = range(5)
MATH_FAST, MATH_EXACT, MATH_AUTO = 0, 1, 2
OK, ERR_ALLOC, ERR_INVALID, ERR_DEVICE = 0, 1, 2, 3

PRECISION_NAMES = {"fp32": 0, "fp16": 1, "bf16": 2, "int8": 3, "int4": 4, "int2": 5}

f32p = C.POINTER(C.c_float)
u32p = C.POINTER(C.c_uint32)
u64p = C.POINTER(C.c_uint64)


class NeuralNetwork(C.Structure):
    _fields_ = [
        ("layers", C.c_uint32), ("topology", u32p), ("act_func", C.POINTER(C.c_int)),
        ("weights", f32p), ("biases", f32p), ("neurons", f32p),
        ("grad_weights", f32p), ("grad_biases", f32p),
        ("opt_m_weights", f32p), ("opt_m_biases", f32p), ("opt_v_weights", f32p), ("opt_v_biases", f32p),
        ("neuron_offsets", u64p), ("weight_offsets", u64p), ("bias_offsets", u64p),
        ("total_neurons", C.c_uint64), ("total_weights", C.c_uint64), ("total_biases", C.c_uint64),
        ("time_step", C.c_uint64), ("loss_func", C.c_int),
    ]


NetP = C.POINTER(NeuralNetwork)
TrainCallback = C.CFUNCTYPE(C.c_bool, NetP, C.c_size_t, C.c_float)
LogCallback = C.CFUNCTYPE(None, C.c_int, C.c_char_p)


class NeuralNetworkArgs(C.Structure):
    _fields_ = [("loss_func", C.c_int)]


class LayerArgs(C.Structure):
    _fields_ = [("net", NetP), ("neurons_amount", C.c_uint32), ("act_func", C.c_int), ("weight_initialization", C.c_int)]


class ForwardArgs(C.Structure):
    _fields_ = [("net", NetP), ("input", f32p)]


class ForwardBatchArgs(C.Structure):
    _fields_ = [("net", NetP), ("inputs", C.c_void_p), ("sample_count", C.c_uint32), ("outputs", C.c_void_p)]


class TrainArgs(C.Structure):
    _fields_ = [
        ("net", NetP), ("training_mode", C.c_int), ("training_strategy", C.c_int), ("optimizer_type", C.c_int),
        ("inputs", C.c_void_p), ("targets", C.c_void_p), ("sample_count", C.c_uint32), ("batch_size", C.c_uint32),
        ("epochs", C.c_size_t),
        ("learning_rate", C.c_float), ("weight_decay", C.c_float), ("momentum", C.c_float), ("beta1", C.c_float),
        ("beta2", C.c_float), ("epsilon", C.c_float), ("max_grad_norm", C.c_float),
        ("reset_optimizer", C.c_bool), ("nan_check_interval", C.c_size_t), ("report_interval", C.c_size_t),
        ("autosave_mode", C.c_int), ("autosave_interval", C.c_size_t), ("autosave_path", C.c_char_p),
        ("autosave_do_not_save_optimizer", C.c_bool), ("autosave_precision", C.c_int),
        ("callback", TrainCallback), ("callback_interval", C.c_size_t),
    ]


class SaveArgs(C.Structure):
    _fields_ = [("net", NetP), ("filename", C.c_char_p), ("do_not_save_optimizer", C.c_bool), ("precision", C.c_int)]


class KLayer(C.Structure):
    """spgk_layer of include/spingalett_b200_kernels.h"""
    _fields_ = [("w", C.c_void_p), ("bias", C.c_void_p), ("w_scale", C.c_float), ("in_", C.c_uint32),
                ("out", C.c_uint32), ("precision", C.c_int32), ("act", C.c_int32), ("bias_absmax", C.c_float)]


# the 21 exported functions of the reference ABI (Spingalett.h:202-238)
REFERENCE_SYMBOLS = [
    "spingalett_last_error_code", "spingalett_last_error_message", "spingalett_clear_error",
    "spingalett_get_compute_mode", "spingalett_set_compute_mode", "spingalett_get_num_threads",
    "spingalett_set_num_threads", "spingalett_set_log_callback", "spingalett_set_log_level",
    "spingalett_set_verbose", "spingalett_get_verbose", "new_spingalett_struct_arguments",
    "layer_struct_arguments", "activate", "derivative", "forward_struct_arguments", "train_struct_arguments",
    "save_spingalett_struct_arguments", "load_spingalett", "print_parameters", "free_network",
]


def bind_reference_abi(lib):
    """Attach argument/return types for the 21 reference functions."""
    lib.spingalett_last_error_code.restype = C.c_int
    lib.spingalett_last_error_message.restype = C.c_char_p
    lib.spingalett_clear_error.restype = None
    lib.spingalett_get_compute_mode.restype = C.c_int
    lib.spingalett_set_compute_mode.argtypes = [C.c_int]
    lib.spingalett_set_compute_mode.restype = None
    lib.spingalett_get_num_threads.restype = C.c_uint
    lib.spingalett_set_num_threads.argtypes = [C.c_uint]
    lib.spingalett_set_num_threads.restype = None
    lib.spingalett_set_log_callback.argtypes = [LogCallback]
    lib.spingalett_set_log_callback.restype = None
    lib.spingalett_set_log_level.argtypes = [C.c_int]
    lib.spingalett_set_log_level.restype = None
    lib.spingalett_set_verbose.argtypes = [C.c_bool]
    lib.spingalett_set_verbose.restype = None
    lib.spingalett_get_verbose.restype = C.c_bool
    lib.new_spingalett_struct_arguments.argtypes = [NeuralNetworkArgs]
    lib.new_spingalett_struct_arguments.restype = NetP
    lib.layer_struct_arguments.argtypes = [LayerArgs]
    lib.layer_struct_arguments.restype = None
    lib.activate.argtypes = [C.c_float, C.c_int]
    lib.activate.restype = C.c_float
    lib.derivative.argtypes = [C.c_float, C.c_int]
    lib.derivative.restype = C.c_float
    lib.forward_struct_arguments.argtypes = [ForwardArgs]
    lib.forward_struct_arguments.restype = f32p
    lib.train_struct_arguments.argtypes = [TrainArgs]
    lib.train_struct_arguments.restype = None
    lib.save_spingalett_struct_arguments.argtypes = [SaveArgs]
    lib.save_spingalett_struct_arguments.restype = None
    lib.load_spingalett.argtypes = [C.c_char_p]
    lib.load_spingalett.restype = NetP
    lib.print_parameters.argtypes = [NetP]
    lib.print_parameters.restype = None
    lib.free_network.argtypes = [NetP]
    lib.free_network.restype = None
    return lib


EXTENSION_SYMBOLS = [
    "forward_batch_struct_arguments", "spingalett_set_math_mode", "spingalett_get_math_mode",
    "spingalett_set_device", "spingalett_get_device_count", "spingalett_set_stream", "spingalett_sync_weights",
    "spingalett_seed", "spingalett_kernel_launches", "spingalett_last_path",
    "spingalett_profile", "spingalett_profile_read", "spingalett_synchronize",
    "spingalett_set_auto_margin", "spingalett_get_auto_margin", "spingalett_last_repaired", "spingalett_net_margin",
    "spingalett_dist_unique_id", "spingalett_dist_init", "spingalett_dist_shutdown", "spingalett_dist_world",
    "spingalett_set_devices", "spingalett_split_rows", "spingalett_dist_agreement_floats", "spingalett_dist_pack_agreement", "spingalett_dist_check_agreement",
]


def bind_extensions(lib):
    lib.forward_batch_struct_arguments.argtypes = [ForwardBatchArgs]
    lib.forward_batch_struct_arguments.restype = C.c_void_p
    lib.spingalett_set_math_mode.argtypes = [C.c_int]
    lib.spingalett_set_math_mode.restype = None
    lib.spingalett_get_math_mode.restype = C.c_int
    lib.spingalett_set_device.argtypes = [C.c_int]
    lib.spingalett_set_device.restype = C.c_int
    lib.spingalett_get_device_count.restype = C.c_int
    lib.spingalett_set_devices.argtypes = [C.POINTER(C.c_int), C.c_int]
    lib.spingalett_set_devices.restype = C.c_int
    lib.spingalett_split_rows.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, u32p, u32p]
    lib.spingalett_split_rows.restype = None
    lib.spingalett_set_stream.argtypes = [NetP, C.c_void_p]
    lib.spingalett_set_stream.restype = None
    lib.spingalett_sync_weights.argtypes = [NetP]
    lib.spingalett_sync_weights.restype = C.c_int
    lib.spingalett_seed.argtypes = [C.c_uint64]
    lib.spingalett_seed.restype = None
    lib.spingalett_kernel_launches.restype = C.c_uint64
    lib.spingalett_last_path.restype = C.c_char_p
    lib.spingalett_set_auto_margin.argtypes = [C.c_float]
    lib.spingalett_set_auto_margin.restype = None
    lib.spingalett_get_auto_margin.restype = C.c_float
    lib.spingalett_last_repaired.argtypes = [NetP]
    lib.spingalett_last_repaired.restype = C.c_uint32
    lib.spingalett_net_margin.argtypes = [NetP]
    lib.spingalett_net_margin.restype = C.c_float
    lib.spingalett_dist_unique_id.argtypes = [C.c_void_p]
    lib.spingalett_dist_unique_id.restype = C.c_int
    lib.spingalett_dist_init.argtypes = [C.c_int, C.c_int, C.c_void_p]
    lib.spingalett_dist_init.restype = C.c_int
    lib.spingalett_dist_shutdown.restype = None
    lib.spingalett_dist_world.restype = C.c_int
    lib.spingalett_dist_agreement_floats.restype = C.c_int
    lib.spingalett_dist_pack_agreement.argtypes = [C.POINTER(TrainArgs), f32p]
    lib.spingalett_dist_pack_agreement.restype = None
    lib.spingalett_dist_check_agreement.argtypes = [f32p, f32p, C.c_int]
    lib.spingalett_dist_check_agreement.restype = C.c_int
    lib.spingalett_synchronize.argtypes = [NetP]
    lib.spingalett_synchronize.restype = C.c_int
    lib.spingalett_profile.argtypes = [NetP, C.c_bool]
    lib.spingalett_profile.restype = None
    lib.spingalett_profile_read.argtypes = [NetP, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]
    lib.spingalett_profile_read.restype = None
    return lib
