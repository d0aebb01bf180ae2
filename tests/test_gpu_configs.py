"""GPU parity on the two large benchmark configurations (seeded synthetic weights of the named
shapes; the oracle checks a bounded number of rows, size-independent properties cover the rest).

  W: 4096-8192-8192-8192-8192-4096(Tanh)-1000(Softmax), LeakyReLU hidden, "Xavier" weights stored BF16,
     N(0,1) inputs, batch 16384 (oracle on 192 rows).
  L: 8192-16384-16384-8192-1000(Softmax), FOO52 hidden, He weights stored INT4, N(0,1) inputs,
     batch 1 / 8 (memory-bound dequant-GEMV) and 64 / 256 (tensor path).
"""
import numpy as np
import pytest

import nets

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def w_net(spg, oracle, has_gpu, tmp_path_factory):
    assert has_gpu, "no CUDA device"
    path = str(tmp_path_factory.mktemp("cfg") / "W_bf16.nn")
    nets.make_net_file(spg, path, nets.W_TOPO, nets.W_ACTS, spg.abi.PRECISION_BFLOAT16, gain=1.0, seed=77)
    net = spg.Network.load(path)
    onet = oracle.OracleNet.from_file(path)
    yield net, onet
    net.free()


@pytest.fixture(scope="module")
def l_net(spg, oracle, has_gpu, tmp_path_factory):
    assert has_gpu, "no CUDA device"
    path = str(tmp_path_factory.mktemp("cfg") / "L_int4.nn")
    nets.make_net_file(spg, path, nets.L_TOPO, nets.L_ACTS, spg.abi.PRECISION_INT4, gain=2.0, seed=78)
    net = spg.Network.load(path)
    onet = oracle.OracleNet.from_file(path)
    yield net, onet
    net.free()


_W_CACHE = {}


def _wide_case(onet):
    """Inputs of the W configuration and the oracle's outputs on 192 of its rows (computed once per session)."""
    if not _W_CACHE:
        n = 16384
        x = nets.normal_inputs(n, nets.W_TOPO[0], seed=5)
        rows = np.random.default_rng(1).choice(n, 192, replace=False)
        _W_CACHE.update(x=x, rows=rows, want=onet.forward_batch(x[rows]))
    return _W_CACHE["x"], _W_CACHE["rows"], _W_CACHE["want"]


@pytest.mark.parametrize("mode", ["exact", "auto", "fast"])
def test_wide_bf16_mlp_batch_16384(spg, w_net, mode):
    """All three math modes on the W configuration against the oracle (bar: 99.9 % argmax, 2e-3).  AUTO, the
    library default, takes the one-term pass plus the exact recomputation of low-margin rows of a 1000-wide softmax."""
    net, onet = w_net
    x, rows, want = _wide_case(onet)
    spg.set_math_mode({"exact": spg.abi.MATH_EXACT, "auto": spg.abi.MATH_AUTO, "fast": spg.abi.MATH_FAST}[mode])
    try:
        got = net.forward_batch(x)
        assert spg.last_path() == "tcgen05"
        agree, err = nets.parity(got[rows], want)
        if mode == "exact":
            assert agree == 1.0 and err <= 2e-5, (agree, err)
        elif mode == "auto":
            assert agree >= 0.999 and err <= 2e-3, (agree, err)
            assert agree == 1.0, agree                               # 192 rows: one flip would already be 0.5 %
            assert spg.lib().spingalett_last_repaired(net._h) > 0     # the margin pass found rows to recompute
        else:
            # one bf16 term per operand: the stated error bar holds, the argmax bar is not promised in this mode
            assert err <= 2e-3 and agree >= 0.97, (agree, err)
        assert np.all(np.isfinite(got)) and np.allclose(got.sum(1), 1.0, atol=1e-4)
        if mode == "exact":
            # rows are independent: the same rows in a small batch give the same result
            again = net.forward_batch(x[rows])
            assert np.abs(again - got[rows]).max() <= 2e-6
    finally:
        spg.set_math_mode(spg.abi.MATH_AUTO)


@pytest.mark.parametrize("n", [1, 8, 20, 64, 128, 256])
def test_large_int4_mlp_batch_sweep(spg, l_net, n):
    net, onet = l_net
    x = nets.normal_inputs(n, nets.L_TOPO[0], seed=100 + n)
    spg.set_math_mode(spg.abi.MATH_EXACT)
    got = net.forward_batch(x)
    # 9..24 rows: GEMV in groups of 8; up to 96 rows: one pass of the streaming kernel; beyond: the GEMM chain on kept operands
    assert spg.last_path() == ("gemv" if n <= 24 else "wstream" if n <= 96 else "tcgen05")
    rows = np.arange(n) if n <= 64 else np.random.default_rng(2).choice(n, 64, replace=False)
    want = onet.forward_batch(x[rows])
    agree, err = nets.parity(got[rows], want)
    assert agree == 1.0 and err <= 2e-5, (n, agree, err)        # bar: 99.9 % / 5e-3
    assert np.allclose(got.sum(1), 1.0, atol=1e-4)
    if n == 1:
        one = net.forward(x[0])                                  # the reference's single-sample entry point
        assert np.abs(one - want[0]).max() <= 2e-5
    if n <= 24:
        # the integer-digit GEMV (default for integer files) against the bf16-term GEMV on the whole chain
        lib = spg.lib()
        lib.spgk_gemv_set_int_path(0)
        try:
            other = net.forward_batch(x)
        finally:
            lib.spgk_gemv_set_int_path(1)
        assert spg.last_path() == "gemv"
        assert np.abs(other - got).max() <= 2e-6, np.abs(other - got).max()


@pytest.mark.parametrize("prec", ["fp16", "bf16", "int8", "int4", "int2"])
def test_save_through_the_device_encoder_writes_the_same_file(spg, has_gpu, tmp_path, prec, monkeypatch):
    """Arrays of a million elements or more are quantised on the GPU by save_spingalett; the file must equal the one
    the host encoder writes."""
    assert has_gpu
    p = {"fp16": 1, "bf16": 2, "int8": 3, "int4": 4, "int2": 5}[prec]
    # 1 134 100 weights in the first matrix: above the threshold, and an odd count for the 4- and 2-bit tails
    net = spg.Network.build([1100, 1031, 10], [spg.abi.ACT_RELU, spg.abi.ACT_SOFTMAX], seed=99)
    a, b = str(tmp_path / "dev.nn"), str(tmp_path / "host.nn")
    net.save(a, p, with_optimizer=True)
    monkeypatch.setenv("SPINGALETT_HOST_ENCODE", "1")
    net.save(b, p, with_optimizer=True)
    monkeypatch.delenv("SPINGALETT_HOST_ENCODE")
    assert open(a, "rb").read() == open(b, "rb").read()
    net.free()


def test_non_finite_input_rows_poison_only_themselves(spg, l_net):
    """An infinity or a NaN in one input row: that row's outputs are not finite (the reference's would not be either),
    every other row of the batch is what it is without the bad row.  Small batch = integer-digit GEMV (the row's
    fixed-point scale becomes NaN), larger batches = the streaming and tensor-core chains."""
    net, _ = l_net
    spg.set_math_mode(spg.abi.MATH_AUTO)
    for n, bad in ((2, 1), (8, 3), (40, 17), (1024, 500)):
        x = nets.normal_inputs(n, nets.L_TOPO[0], seed=300 + n)
        clean = net.forward_batch(x)
        y = x.copy()
        y[bad, 5] = np.inf
        y[bad, 77] = np.nan
        got = net.forward_batch(y)
        good = np.arange(n) != bad
        assert not np.any(np.isfinite(got[bad])), (n, spg.last_path(), got[bad][:4])
        assert np.all(np.isfinite(got[good]))
        assert np.abs(got[good] - clean[good]).max() <= 2e-6, (n, spg.last_path())
