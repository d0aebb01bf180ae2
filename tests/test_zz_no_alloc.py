"""The allocation-free layer entry point (spgk_layer_gemm_tc_noalloc) against the
regular one (spgk_layer_gemm_tc with caller-allocated scratch), through the C ABI.

Some users of this library may not allocate device memory while serving -- their
process handed all of HBM to its own arena at start-up, or they cannot afford the
device-wide synchronisation inside cudaMalloc -- so this variant keeps its scratch
(the expanded 16-bit weight operand and the kernel's status word) in a fixed array
of the library's device image.  Both entry points run the same kernels on the same
operands, so their outputs must be identical (and both are held to a float64
product of the same operands); two calls in a row with different layers check that
nothing left in the shared array by the first call leaks into the second.  The file
sorts last so that a run stopping at the first failure has already run every other test; it also passes on its own in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _bind(spg):
    lib = spg.lib()
    vp = C.c_void_p
    lib.spgk_error_string.restype = C.c_char_p
    lib.spgk_split16.argtypes = [vp, C.c_uint32, C.c_uint32, C.c_uint32, vp, C.c_uint32, C.c_uint64, C.c_int, C.c_int, vp]
    lib.spgk_dequant16.argtypes = [C.POINTER(spg.abi.KLayer), vp, C.c_uint32, C.c_uint64, C.c_int, C.c_int, vp]
    lib.spgk_layer_gemm_tc.argtypes = [C.POINTER(spg.abi.KLayer), vp, C.c_uint32, C.c_uint64, C.c_int, C.c_int,
                                       vp, C.c_uint32, C.c_uint64, C.c_int, C.c_int,
                                       vp, C.c_uint32, C.c_uint64, C.c_int, vp, C.c_uint32,
                                       C.c_uint32, C.c_int, vp, vp]
    lib.spgk_gemm_tc_status.argtypes = [vp, vp]
    lib.spgk_layer_gemm_tc_noalloc.argtypes = [C.POINTER(spg.abi.KLayer), vp, C.c_uint32, C.c_uint64, C.c_int, C.c_int,
                                               vp, C.c_uint32, C.c_uint64, C.c_int, vp, C.c_uint32,
                                               C.c_uint32, C.c_int, vp]
    lib.spgk_weights16_bytes.argtypes = [C.POINTER(spg.abi.KLayer), C.c_int]
    lib.spgk_weights16_bytes.restype = C.c_size_t
    return lib


def _one_layer(spg, lib, oracle, torch, M, N, K, prec, act, parts, seed):
    """Runs one layer through both entry points; returns (regular fp32, no-alloc fp32, regular 16-bit, no-alloc 16-bit)."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(N * K) / np.sqrt(K)).astype(np.float32)
    raw = oracle.Oracle.encode(w, prec)
    skip = 4 if prec >= 3 else 0
    amax = float(np.frombuffer(raw[:4].tobytes(), np.float32)[0]) if skip else 1.0
    scale = amax / {3: 127.0, 4: 7.0, 5: 1.0}[prec] if skip else 1.0
    payload = torch.from_numpy(np.concatenate([raw[skip:], np.zeros(256, np.uint8)])).cuda()
    bias = torch.from_numpy(rng.standard_normal(N).astype(np.float32) * 0.1).cuda()
    L = spg.abi.KLayer(payload.data_ptr(), bias.data_ptr(), scale, K, N, prec, act)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda()
    ld, ldo = (K + 7) & ~7, (N + 7) & ~7
    t16, dt = 1, torch.bfloat16
    a16 = torch.zeros((parts, M, ld), dtype=dt, device="cuda")
    assert lib.spgk_split16(x.data_ptr(), K, M, K, a16.data_ptr(), ld, M * ld, parts, t16, None) == 0
    w_parts = 2 if (prec == 0 and parts == 2) else 1

    # regular entry point: scratch allocated by the caller (here: by torch)
    w16 = torch.zeros((w_parts, N, ld), dtype=dt, device="cuda")
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    ref16 = torch.zeros((parts, M, ldo), dtype=dt, device="cuda")
    ref32 = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    assert lib.spgk_dequant16(C.byref(L), w16.data_ptr(), ld, N * ld, w_parts, t16, None) == 0
    rc = lib.spgk_layer_gemm_tc(C.byref(L), w16.data_ptr(), ld, N * ld, w_parts, t16, a16.data_ptr(), ld, M * ld, parts, t16,
                                ref16.data_ptr(), ldo, M * ldo, parts, ref32.data_ptr(), N, M, 0, status.data_ptr(), None)
    assert rc == 0, lib.spgk_error_string()
    assert lib.spgk_gemm_tc_status(status.data_ptr(), None) == 0

    # allocation-free entry point: same inputs and outputs, scratch inside the library
    got16 = torch.zeros((parts, M, ldo), dtype=dt, device="cuda")
    got32 = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    rc = lib.spgk_layer_gemm_tc_noalloc(C.byref(L), a16.data_ptr(), ld, M * ld, parts, t16,
                                        got16.data_ptr(), ldo, M * ldo, parts, got32.data_ptr(), N, M, 0, None)
    assert rc == 0, lib.spgk_error_string()
    # Both results are also held to a float64 product of the operands the tensor cores saw (the rounded activation terms
    # and the decoded weights), so the two entry points cannot agree on a wrong answer.
    if prec == 0:
        dec = w16.float().cpu().numpy()[:, :, :K].astype(np.float64).sum(0)   # the bf16 terms of the fp32 weights
    else:
        dec = oracle.Oracle.decode(raw, N * K, prec).astype(np.float64).reshape(N, K)
    xs = a16.float().cpu().numpy()[:, :, :K].astype(np.float64).sum(0)
    z = xs @ dec.T + bias.cpu().numpy().astype(np.float64)
    want = {1: lambda v: np.maximum(v, 0), 3: lambda v: np.where(v > 0, v, 0.01 * v),
            4: lambda v: np.where(v > 1, 1 + 0.01 * (v - 1), np.where(v < 0, 0.01 * v, v))}[act](z)
    tol = (2e-5 * np.sqrt(K) + 1e-5) * max(1.0, np.abs(want).max())
    for name, res in (("regular", ref32), ("no-alloc", got32)):
        err = np.abs(res.cpu().numpy() - want).max()
        assert err <= tol, (name, err, tol)
    return ref32.cpu().numpy(), got32.cpu().numpy(), ref16.float().cpu().numpy(), got16.float().cpu().numpy()


def test_noalloc_entry_point_matches_regular_one_twice_in_a_row(spg, oracle, has_gpu):
    assert has_gpu, "no CUDA device"
    import torch
    lib = _bind(spg)
    # first call: a wide INT4 layer fills most of the columns of the shared array ...
    r32, g32, r16, g16 = _one_layer(spg, lib, oracle, torch, M=777, N=1000, K=512, prec=4, act=1, parts=2, seed=1)
    assert np.isfinite(r32).all() and np.abs(r32).max() > 0
    assert np.array_equal(g32, r32) and np.array_equal(g16, r16)
    # ... second call: a smaller FP32 layer (two weight planes) that would read stale data if any survived
    r32, g32, r16, g16 = _one_layer(spg, lib, oracle, torch, M=300, N=40, K=100, prec=0, act=3, parts=2, seed=2)
    assert np.abs(r32).max() > 0
    assert np.array_equal(g32, r32) and np.array_equal(g16, r16)
    # and the first shape once more, one activation term
    r32, g32, r16, g16 = _one_layer(spg, lib, oracle, torch, M=129, N=264, K=136, prec=3, act=4, parts=1, seed=3)
    assert np.array_equal(g32, r32) and np.array_equal(g16, r16)


def test_noalloc_entry_point_refuses_layers_beyond_its_array(spg, has_gpu):
    assert has_gpu, "no CUDA device"
    import torch
    lib = _bind(spg)
    N, K = 4096, 2048                       # 16 MiB as a 16-bit operand: over the 8 MiB the library carries
    payload = torch.zeros(N * K + 256, dtype=torch.uint8, device="cuda")
    bias = torch.zeros(N, device="cuda")
    L = spg.abi.KLayer(payload.data_ptr(), bias.data_ptr(), 1.0, K, N, 3, 1)
    assert lib.spgk_weights16_bytes(C.byref(L), 1) > (8 << 20)
    a16 = torch.zeros((1, 128, K), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((128, N), device="cuda")
    rc = lib.spgk_layer_gemm_tc_noalloc(C.byref(L), a16.data_ptr(), K, 128 * K, 1, 1, None, 0, 0, 1,
                                        out.data_ptr(), N, 128, 0, None)
    assert rc == -2                         # SPGK_E_ARG
    msg = lib.spgk_error_string().decode()
    assert "built-in array" in msg and str(8 << 20) in msg
