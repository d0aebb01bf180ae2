"""Host-side checks that need no GPU: the shared library loads, exports every
declared symbol, keeps the reference's record layouts and error behaviour, and
reads/writes .nn files identically to the reference (golden fixtures)."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

from conftest import PRECS, ROOT, golden, ulp_diff

META = json.load(open(golden("golden.json")))


def _declared(header, macro):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = "\n".join(l for l in text.splitlines() if not l.lstrip().startswith("#"))
    names = re.findall(macro + r"\s+[^;(]*?\b(\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol(spg):
    lib = spg.lib()
    public = _declared("spingalett_b200.h", "SPINGALETT_API")
    kernels = _declared("spingalett_b200_kernels.h", "SPGK_API")
    assert len(public) >= 31 and len(kernels) >= 20
    for name in public + kernels:
        assert hasattr(lib, name), name
    for name in spg.abi.REFERENCE_SYMBOLS:
        assert name in public


def test_record_layouts_match_reference_abi(spg):
    a = spg.abi
    # sizes/offsets of Include/Spingalett/Spingalett.h on x86-64 SysV
    assert C.sizeof(a.NeuralNetwork) == 160
    assert a.NeuralNetwork.weights.offset == 24 and a.NeuralNetwork.neurons.offset == 40
    assert a.NeuralNetwork.neuron_offsets.offset == 96 and a.NeuralNetwork.total_neurons.offset == 120
    assert a.NeuralNetwork.time_step.offset == 144 and a.NeuralNetwork.loss_func.offset == 152
    assert C.sizeof(a.LayerArgs) == 24 and C.sizeof(a.ForwardArgs) == 16
    assert C.sizeof(a.TrainArgs) == 152 and C.sizeof(a.SaveArgs) == 24


def test_header_compiles_as_c23_and_cxx(tmp_path):
    import subprocess
    src = tmp_path / "t.c"
    src.write_text('#include <Spingalett/Spingalett.h>\n_Static_assert(sizeof(NeuralNetwork)==160,"");\n'
                   '_Static_assert(sizeof(TrainArgs)==152,"");\nint main(void){NeuralNetwork*n=new_spingalett(.loss_func=LOSS_CROSS_ENTROPY);'
                   'layer(n,4);layer(.net=n,.neurons_amount=2,.act_func=ACT_SOFTMAX);(void)forward(n,0);return 0;}\n')
    subprocess.run(["gcc", "-std=c2x", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)], check=True)
    cxx = tmp_path / "t.cpp"
    cxx.write_text('#include <Spingalett/Spingalett.h>\n#include <spingalett_b200_kernels.h>\nint main(){return 0;}\n')
    subprocess.run(["g++", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(cxx)], check=True)


def test_settings_roundtrip(spg):
    lib = spg.lib()
    lib.spingalett_set_compute_mode(spg.abi.COMPUTE_OPENBLAS)
    assert lib.spingalett_get_compute_mode() == spg.abi.COMPUTE_OPENBLAS
    lib.spingalett_set_compute_mode(99)            # out of range: ignored (reference Settings.c:26-29)
    assert lib.spingalett_get_compute_mode() == spg.abi.COMPUTE_OPENBLAS
    lib.spingalett_set_compute_mode(spg.abi.COMPUTE_SINGLE_THREADED)
    lib.spingalett_set_num_threads(5)
    assert lib.spingalett_get_num_threads() == 5
    lib.spingalett_set_verbose(True)
    assert lib.spingalett_get_verbose()
    lib.spingalett_set_verbose(False)
    seen = []
    cb = spg.abi.LogCallback(lambda lvl, msg: seen.append((lvl, msg)))
    lib.spingalett_set_log_callback(cb)
    lib.spingalett_set_log_level(spg.abi.LOG_DEBUG)
    lib.spingalett_set_verbose(True)
    n = spg.Network.new(spg.abi.LOSS_MSE)
    n.free()
    lib.spingalett_set_verbose(False)
    lib.spingalett_set_log_callback(spg.abi.LogCallback())
    lib.spingalett_set_log_level(spg.abi.LOG_INFO)
    assert any(b"Creating new network" in m for _, m in seen)


def test_error_convention(spg):
    lib, a = spg.lib(), spg.abi
    assert lib.spingalett_last_error_code() == a.OK
    # invalid loss -> NULL + ERR_INVALID (reference Network.c:36-39)
    assert not lib.new_spingalett_struct_arguments(a.NeuralNetworkArgs(7))
    assert lib.spingalett_last_error_code() == a.ERR_INVALID
    assert b"loss" in lib.spingalett_last_error_message().lower()
    lib.spingalett_clear_error()
    assert lib.spingalett_last_error_code() == a.OK and lib.spingalett_last_error_message() == b""
    net = lib.new_spingalett_struct_arguments(a.NeuralNetworkArgs(a.LOSS_MSE))
    lib.layer_struct_arguments(a.LayerArgs(net, 0, 0, 0))        # 0 neurons (Network.c:53-56)
    assert lib.spingalett_last_error_code() == a.ERR_INVALID
    lib.spingalett_clear_error()
    lib.layer_struct_arguments(a.LayerArgs(net, 3, 0, 0))
    lib.layer_struct_arguments(a.LayerArgs(net, 2, 55, 0))       # bad activation
    assert lib.spingalett_last_error_code() == a.ERR_INVALID
    lib.spingalett_clear_error()
    lib.layer_struct_arguments(a.LayerArgs(net, 2, a.ACT_RELU, 55))   # bad init
    assert lib.spingalett_last_error_code() == a.ERR_INVALID
    lib.spingalett_clear_error()
    # forward(NULL, ...) and forward(net, NULL) return NULL WITHOUT an error (Network.c:207)
    x = (C.c_float * 3)()
    assert not lib.forward_struct_arguments(a.ForwardArgs(None, x))
    assert not lib.forward_struct_arguments(a.ForwardArgs(net, None))
    assert lib.spingalett_last_error_code() == a.OK
    # fewer than two layers -> ERR_INVALID (Network.c:209-212)
    assert not lib.forward_struct_arguments(a.ForwardArgs(net, x))
    assert lib.spingalett_last_error_code() == a.ERR_INVALID
    lib.spingalett_clear_error()
    lib.free_network(net)
    lib.free_network(None)                                        # NULL-safe (Network.c:284)
    lib.save_spingalett_struct_arguments(a.SaveArgs(None, b"x", True, 0))
    assert lib.spingalett_last_error_code() == a.ERR_INVALID
    lib.spingalett_clear_error()
    assert not lib.load_spingalett(None)
    assert lib.spingalett_last_error_code() == a.ERR_INVALID
    lib.spingalett_clear_error()
    assert not lib.load_spingalett(b"/nonexistent/file.nn")
    assert lib.spingalett_last_error_code() == a.ERR_INVALID


def test_layer_builds_reference_layout(spg):
    net = spg.Network.build([5, 4, 3], [spg.abi.ACT_RELU, spg.abi.ACT_SOFTMAX], spg.abi.WEIGHT_INITIALIZATION_NONE)
    c = net.c
    assert c.layers == 3 and c.total_weights == 32 and c.total_biases == 7 and c.total_neurons == 12
    assert [c.neuron_offsets[i] for i in range(4)] == [0, 5, 9, 12]
    assert [c.weight_offsets[i] for i in range(2)] == [0, 20] and [c.bias_offsets[i] for i in range(2)] == [0, 4]
    assert not c.grad_weights          # created by the first train() call only
    assert np.all(net.weights == 0)
    net.free()


def test_seeded_init_reproduces_reference_stream(spg):
    """layer(..HE) after spingalett_seed(s) draws the weights the reference draws after rng_seed(s)."""
    m = META["nets"]["small"]
    net = spg.Network.build(m["topology"], m["acts"], m["init"], seed=m["seed"])
    ref = np.load(golden("small.fp32.weights.npy"))[: net.c.total_weights]
    assert ulp_diff(net.weights, ref) <= 1
    assert np.array_equal(net.weights, ref) or np.mean(net.weights != ref) < 0.01
    net.free()
    m = META["nets"]["wide8"]                       # U(-1,1) initialisation
    net = spg.Network.build(m["topology"], m["acts"], m["init"], seed=m["seed"])
    ref = np.load(golden("wide8.fp32.weights.npy"))[: net.c.total_weights]
    assert np.array_equal(net.weights, ref)
    net.free()


@pytest.mark.parametrize("name", list(META["nets"].keys()))
@pytest.mark.parametrize("prec", PRECS)
def test_load_fills_fp32_mirror_like_reference(spg, name, prec):
    net = spg.Network.load(golden(f"{name}.{prec}.nn"))
    ref = np.load(golden(f"{name}.{prec}.weights.npy"))
    got = np.concatenate([net.weights, net.biases])
    assert ulp_diff(got, ref) <= (1 if prec in ("int8", "int4") else 0)
    assert net.topology == META["nets"][name]["topology"] and net.acts == META["nets"][name]["acts"]
    net.free()


@pytest.mark.parametrize("name", list(META["nets"].keys()))
@pytest.mark.parametrize("prec", PRECS)
def test_save_is_byte_identical_to_reference(spg, tmp_path, name, prec):
    src = spg.Network.load(golden(f"{name}.fp32.nn"))
    out = tmp_path / f"{name}_{prec}"                     # no extension: ".nn" gets appended
    src.save(str(out), PRECS.index(prec))
    want = open(golden(f"{name}.{prec}.nn"), "rb").read()
    got = open(str(out) + ".nn", "rb").read()
    assert got == want
    src.free()


def test_optimizer_sections_roundtrip(spg, tmp_path):
    for prec in ("fp32", "int8"):
        net = spg.Network.load(golden(f"withopt.{prec}.nn"))
        st = np.load(golden(f"withopt.{prec}.state.npz"))
        c = net.c
        assert c.time_step == 42
        for field, key, n in [("opt_m_weights", "m_w", c.total_weights), ("opt_v_weights", "v_w", c.total_weights),
                              ("opt_m_biases", "m_b", c.total_biases), ("opt_v_biases", "v_b", c.total_biases)]:
            got = np.ctypeslib.as_array(getattr(c, field), shape=(n,))
            assert ulp_diff(got, st[key]) <= 1
        if prec == "fp32":
            out = tmp_path / "again.nn"
            net.save(str(out), 0, with_optimizer=True)
            assert open(out, "rb").read() == open(golden("withopt.fp32.nn"), "rb").read()
        net.free()


def test_load_rejects_corrupt_headers(spg, tmp_path):
    lib, a = spg.lib(), spg.abi
    raw = open(golden("small.int8.nn"), "rb").read()
    header = 2 + 4 + 1 + 1 + 1 + 16 + 3
    path = tmp_path / "t.nn"
    for cut in range(header):                          # short read in every header field
        path.write_bytes(raw[:cut])
        assert not lib.load_spingalett(str(path).encode())
        assert lib.spingalett_last_error_code() == a.ERR_INVALID
        lib.spingalett_clear_error()
    for offset, value in [(0, 2), (2, 1), (6, 5), (8, 9), (9 + 16, 200)]:   # version, layers<2, loss, precision, activation
        bad = bytearray(raw)
        bad[offset] = value
        if offset == 2:
            bad[2:6] = (1).to_bytes(4, "little")
        path.write_bytes(bytes(bad))
        assert not lib.load_spingalett(str(path).encode()), offset
        assert lib.spingalett_last_error_code() == a.ERR_INVALID
        lib.spingalett_clear_error()
    # zero-width layer is refused by layer() (Network.c:53-56) and so by load
    bad = bytearray(raw)
    bad[9 + 4:9 + 8] = (0).to_bytes(4, "little")
    path.write_bytes(bytes(bad))
    assert not lib.load_spingalett(str(path).encode())
    lib.spingalett_clear_error()


def test_truncated_payload_returns_partial_net_with_error(spg, tmp_path):
    """Serialize.c:596-608: a short payload sets ERR_INVALID but the net is still returned."""
    lib, a = spg.lib(), spg.abi
    raw = open(golden("small.fp32.nn"), "rb").read()
    path = tmp_path / "short.nn"
    path.write_bytes(raw[: len(raw) - 50])
    h = lib.load_spingalett(str(path).encode())
    assert h and lib.spingalett_last_error_code() == a.ERR_INVALID
    full = np.load(golden("small.fp32.weights.npy"))
    got = np.ctypeslib.as_array(h.contents.weights, shape=(h.contents.total_weights,))
    first = 20 * 33
    assert np.array_equal(got[:first], full[:first])
    lib.spingalett_clear_error()
    lib.free_network(h)


def test_stale_error_makes_load_fail(spg):
    """The error state is sticky and load checks it after each layer (Serialize.c:556)."""
    lib, a = spg.lib(), spg.abi
    lib.new_spingalett_struct_arguments(a.NeuralNetworkArgs(9))        # leaves ERR_INVALID pending
    assert not lib.load_spingalett(golden("small.fp32.nn").encode())
    lib.spingalett_clear_error()
    h = lib.load_spingalett(golden("small.fp32.nn").encode())
    assert h
    lib.free_network(h)


def test_scalar_activation_exports(spg):
    g = np.load(golden("activations.npz"))
    lib = spg.lib()
    for act in range(g["activate"].shape[0]):
        for i, x in enumerate(g["x"]):
            for fn, tab in ((lib.activate, "activate"), (lib.derivative, "derivative")):
                got, want = float(np.float32(fn(float(x), act))), float(g[tab][act, i])
                if np.isnan(want):
                    assert np.isnan(got)
                elif np.isinf(want) or got == want:
                    assert got == want
                else:
                    assert abs(got - want) <= 1e-6 * max(1.0, abs(want))


def test_compute_without_gpu_fails_loudly(spg, has_gpu):
    """No CPU fallback: with no CUDA device every compute entry point reports ERR_DEVICE."""
    if has_gpu:
        pytest.skip("a CUDA device is present")
    net = spg.Network.load(golden("small.fp32.nn"))
    with pytest.raises(spg.SpingalettError) as e:
        net.forward(np.zeros(20, np.float32))
    assert e.value.code == spg.abi.ERR_DEVICE
    with pytest.raises(spg.SpingalettError) as e:
        net.forward_batch(np.zeros((4, 20), np.float32))
    assert e.value.code == spg.abi.ERR_DEVICE
    net.free()


def test_product_does_not_reach_for_the_oracle(spg):
    """Nothing in the shipped package or library imports, links or names the test oracle."""
    pkg = os.path.join(ROOT, "spingalett_b200")
    for base, _, files in os.walk(pkg):
        if os.sep + "build" in base:
            continue
        for f in files:
            if f.endswith((".py", ".c", ".h", ".cu", ".cuh")):
                text = open(os.path.join(base, f), errors="replace").read()
                assert "spg_oracle" not in text and "import oracle" not in text and "from oracle" not in text, f
    import subprocess
    deps = subprocess.run(["ldd", spg.LIB_PATH], capture_output=True, text=True).stdout
    assert "oracle" not in deps and "spingalett_ref" not in deps


@pytest.mark.parametrize("example", ["XOR.c", "Benchmark.c"])
def test_reference_examples_compile_unmodified_against_the_header(spg, tmp_path, example):
    """Where a checkout of the reference is at hand, its example programs compile and link, unmodified, against include/ and
    the library (they are run on a GPU by hand or by tests/c/xor_program.c's test; here only the build is checked)."""
    import subprocess
    from oracle import reference_root
    src = os.path.join(reference_root(), "Examples", example)
    if not os.path.exists(src):
        pytest.skip("no checkout of the reference here")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    libdir = os.path.dirname(spg.LIB_PATH)
    r = subprocess.run(["gcc", "-std=c2x", "-O1", "-I", os.path.join(root, "include"), src, "-o", str(tmp_path / "example"),
                        "-L", libdir, "-lspingalett", "-lm", "-Wl,-rpath," + libdir], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_rank_agreement_check_detects_any_differing_argument(spg):
    """The data-parallel train() refuses to start unless every rank packed the same arguments: the packed bytes summed over
    ranks must equal world times the own bytes (and likewise their squares)."""
    import ctypes as C
    lib, a = spg.lib(), spg.abi
    n = lib.spingalett_dist_agreement_floats()

    def pack(**kw):
        args = a.TrainArgs()
        args.sample_count, args.batch_size, args.epochs = 5120, 256, 100
        args.training_strategy, args.optimizer_type = a.STRATEGY_SMALL_BATCH, a.OPTIMIZER_ADAM
        for k, v in kw.items():
            setattr(args, k, v)
        buf = np.zeros(n, np.float32)
        lib.spingalett_dist_pack_agreement(C.byref(args), buf.ctypes.data_as(a.f32p))
        return buf
    base = pack()
    fp = lambda v: v.ctypes.data_as(a.f32p)
    for world in (2, 3, 8):
        assert lib.spingalett_dist_check_agreement(fp(base * world), fp(base), world) == 1
    for kw in (dict(sample_count=5121), dict(batch_size=128), dict(epochs=101), dict(optimizer_type=a.OPTIMIZER_SGD),
               dict(training_strategy=a.STRATEGY_FULL_BATCH), dict(nan_check_interval=3), dict(max_grad_norm=1.0)):
        other = pack(**kw)
        summed = base + other
        assert lib.spingalett_dist_check_agreement(fp(summed), fp(base), 2) == 0, kw
        assert lib.spingalett_dist_check_agreement(fp(summed), fp(other), 2) == 0, kw
    # three ranks whose values average to the own value still fail (the squares do not)
    lo, mid, hi = pack(sample_count=5119), pack(sample_count=5120), pack(sample_count=5121)
    assert lib.spingalett_dist_check_agreement(fp(lo + mid + hi), fp(mid), 3) == 0


def test_once_per_device_bookkeeping_of_the_launchers(spg):
    """cudaFuncSetAttribute is per device: the launchers run their set-up once per device index, retry a set-up that failed,
    and refuse indices outside the table (host-only check of that bookkeeping)."""
    lib = spg.lib()
    assert lib.spgk_selftest_once_per_device(1, 5, -1) == 1
    assert lib.spgk_selftest_once_per_device(8, 3, -1) == 8          # eight devices, three rounds of calls: eight set-ups
    assert lib.spgk_selftest_once_per_device(4, 3, 2) == 5           # device 2 failed once and was set up again


def test_rendezvous_timeout_wrapper(spg):
    """The communicator rendezvous runs under a host timeout: a call that answers in time passes its result through, one
    that does not (a rank that never joined) ends with SPGK_E_TIMEOUT after the limit instead of blocking for ever."""
    import time
    lib = spg.lib()
    assert lib.spgk_selftest_timed_call(5, 2000) == 0
    t0 = time.time()
    assert lib.spgk_selftest_timed_call(5000, 150) == -4             # SPGK_E_TIMEOUT
    assert time.time() - t0 < 2.0


def test_row_shares_of_the_device_fan_out_cover_the_batch_once(spg):
    """spingalett_split_rows: contiguous shares, sizes within one row of each other, every row exactly once -- also when
    there are fewer rows than shares."""
    import ctypes as C
    lib = spg.lib()
    for rows in (0, 1, 7, 8, 65536, 65537, 1000003):
        for shares in (1, 2, 3, 4, 8, 16):
            spans = []
            for g in range(shares):
                lo, hi = C.c_uint32(), C.c_uint32()
                lib.spingalett_split_rows(rows, shares, g, C.byref(lo), C.byref(hi))
                spans.append((lo.value, hi.value))
            assert spans[0][0] == 0 and spans[-1][1] == rows
            assert all(spans[i][1] == spans[i + 1][0] for i in range(shares - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
            assert spans == [spg.shard_rows(rows, shares, g) for g in range(shares)]
    assert lib.spingalett_set_devices(None, 0) == 0
