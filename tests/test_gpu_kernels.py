"""Kernel-level GPU tests through the spgk_* shim: each hand-written kernel
against a numpy restatement of the same arithmetic on the same operands."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k(spg, has_gpu):
    assert has_gpu, "no CUDA device"
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
    lib.spgk_layer_simt.argtypes = [C.POINTER(spg.abi.KLayer), vp, C.c_uint32, vp, C.c_uint32, C.c_uint32, vp]
    lib.spgk_softmax_rows.argtypes = [vp, C.c_uint32, C.c_uint32, C.c_uint32, vp]
    lib.spgk_layer_gemv.argtypes = [C.POINTER(spg.abi.KLayer), vp, C.c_uint32, vp, C.c_uint32, C.c_uint32, vp, vp]
    lib.spgk_gemv_scratch_bytes.argtypes = [C.POINTER(spg.abi.KLayer), C.c_uint32]
    lib.spgk_gemv_scratch_bytes.restype = C.c_size_t
    lib.spgk_gemv_set_int_path.argtypes = [C.c_int]
    return lib


def _round16(x, t):
    import torch
    dt = torch.float16 if t == 0 else torch.bfloat16
    return torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(dt).float().numpy()


def _softmax(v):
    e = np.exp(v - v.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


ACT = {1: lambda v: np.maximum(v, 0), 6: lambda v: v, 3: lambda v: np.where(v > 0, v, 0.01 * v), 5: _softmax,
       2: np.tanh, 0: lambda v: 1 / (1 + np.exp(-v)),
       4: lambda v: np.where(v > 1, 1 + 0.01 * (v - 1), np.where(v < 0, 0.01 * v, v))}


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 16, 64), (256, 512, 784), (300, 1000, 512), (1000, 10, 1000),
                                   (77, 33, 20), (129, 264, 136), (4096, 512, 784), (128, 256, 8192)])
@pytest.mark.parametrize("t16", [0, 1])
@pytest.mark.parametrize("parts", [1, 2])
def test_gemm_tc_against_numpy(spg, k, M, N, K, t16, parts):
    """tcgen05 GEMM + fused epilogue vs float64 matmul of the same rounded operands."""
    import torch
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32) * 0.1
    act = [1, 6, 3, 2, 0, 4][(M + N + K) % 6]
    scale = 0.75
    ld = (K + 7) & ~7
    ldo = (N + 7) & ~7
    dt = torch.float16 if t16 == 0 else torch.bfloat16
    xd = torch.from_numpy(x).cuda()
    a16 = torch.zeros((parts, M, ld), dtype=dt, device="cuda")
    assert k.spgk_split16(xd.data_ptr(), K, M, K, a16.data_ptr(), ld, M * ld, parts, t16, None) == 0, k.spgk_error_string()
    wd = torch.from_numpy(w).cuda()
    bd = torch.from_numpy(bias).cuda()
    L = spg.abi.KLayer(wd.data_ptr(), bd.data_ptr(), scale, K, N, 0, act)
    w16 = torch.zeros((1, N, ld), dtype=dt, device="cuda")
    assert k.spgk_dequant16(C.byref(L), w16.data_ptr(), ld, N * ld, 1, t16, None) == 0, k.spgk_error_string()
    o16 = torch.full((parts, M, ldo), 7.0, dtype=dt, device="cuda")
    o32 = torch.full((M + 1, N), -3.0, dtype=torch.float32, device="cuda")
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = k.spgk_layer_gemm_tc(C.byref(L), w16.data_ptr(), ld, N * ld, 1, t16, a16.data_ptr(), ld, M * ld, parts, t16,
                              o16.data_ptr(), ldo, M * ldo, parts, o32.data_ptr(), N, M, 0, status.data_ptr(), None)
    assert rc == 0, k.spgk_error_string()
    assert k.spgk_gemm_tc_status(status.data_ptr(), None) == 0, k.spgk_error_string()
    # the operands the tensor cores saw
    xs = a16.float().cpu().numpy()[:, :, :K].astype(np.float64).sum(0)
    ws = w16.float().cpu().numpy()[0, :, :K].astype(np.float64)
    want = ACT[act](xs @ ws.T * scale + bias)
    got = o32.cpu().numpy()
    assert np.all(got[M] == -3.0)                                   # guard row untouched
    tol = 2e-5 * np.sqrt(K) + 1e-5
    assert np.abs(got[:M] - want).max() <= tol * max(1.0, np.abs(want).max()), np.abs(got[:M] - want).max()
    # 16-bit planes reassemble the fp32 result to the precision of the split
    rec = o16.float().cpu().numpy()[:, :, :N].astype(np.float64).sum(0)
    eps = (2.0 ** -11 if t16 == 0 else 2.0 ** -8) ** parts
    assert np.abs(rec - got[:M]).max() <= 1.01 * eps * max(1.0, np.abs(got[:M]).max())


@pytest.mark.parametrize("M,N,K", [(128, 10, 1000), (500, 256, 64), (130, 100, 200)])
def test_gemm_tc_fused_softmax(spg, k, M, N, K):
    import torch
    rng = np.random.default_rng(5)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 2 / np.sqrt(K)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    ld = (K + 7) & ~7
    xd = torch.from_numpy(x).cuda()
    a16 = torch.zeros((2, M, ld), dtype=torch.bfloat16, device="cuda")
    assert k.spgk_split16(xd.data_ptr(), K, M, K, a16.data_ptr(), ld, M * ld, 2, 1, None) == 0
    wd, bd = torch.from_numpy(w).cuda(), torch.from_numpy(bias).cuda()
    L = spg.abi.KLayer(wd.data_ptr(), bd.data_ptr(), 1.0, K, N, 0, 5)
    w16 = torch.zeros((2, N, ld), dtype=torch.bfloat16, device="cuda")
    assert k.spgk_dequant16(C.byref(L), w16.data_ptr(), ld, N * ld, 2, 1, None) == 0
    o32 = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = k.spgk_layer_gemm_tc(C.byref(L), w16.data_ptr(), ld, N * ld, 2, 1, a16.data_ptr(), ld, M * ld, 2, 1,
                              None, 0, 0, 1, o32.data_ptr(), N, M, 1, status.data_ptr(), None)
    assert rc == 0, k.spgk_error_string()
    assert k.spgk_gemm_tc_status(status.data_ptr(), None) == 0
    z = x.astype(np.float64) @ w.astype(np.float64).T + bias
    e = np.exp(z - z.max(1, keepdims=True))
    want = e / e.sum(1, keepdims=True)
    assert np.abs(o32.cpu().numpy() - want).max() < 2e-4


@pytest.mark.parametrize("prec,bits", [(3, 8), (4, 4), (5, 2), (0, 32), (1, 16), (2, 16)])
@pytest.mark.parametrize("out_in", [(33, 20), (9, 15), (7, 9), (256, 64)])
def test_dequant16_every_precision(spg, k, oracle, prec, bits, out_in):
    """Packed payload -> 16-bit operand planes reproduces the stored integers / floats."""
    import torch
    out, inn = out_in
    rng = np.random.default_rng(out * 100 + inn)
    vals = rng.standard_normal(out * inn).astype(np.float32)
    raw = oracle.Oracle.encode(vals, prec)
    dec = oracle.Oracle.decode(raw, out * inn, prec)
    skip = 4 if prec >= 3 else 0
    amax = np.frombuffer(raw[:4].tobytes(), np.float32)[0] if skip else 1.0
    q = {3: 127.0, 4: 7.0, 5: 1.0}.get(prec, 1.0)
    scale = amax / q if skip else 1.0
    payload = torch.from_numpy(np.concatenate([raw[skip:], np.zeros(64, np.uint8)])).cuda()
    L = spg.abi.KLayer(payload.data_ptr(), None, scale, inn, out, prec, 6)
    ld = (inn + 7) & ~7
    for t16, dt in ((0, torch.float16), (1, torch.bfloat16)):
        w16 = torch.full((2, out, ld), 9.0, dtype=dt, device="cuda")
        assert k.spgk_dequant16(C.byref(L), w16.data_ptr(), ld, out * ld, 2, t16, None) == 0
        got = w16.float().cpu().numpy().astype(np.float64)
        assert np.all(got[:, :, inn:] == 0)
        rec = got[:, :, :inn].sum(0).reshape(-1) * scale
        tol = 0 if prec >= 3 or (prec == 1 and t16 == 0) or (prec == 2 and t16 == 1) else 2.0 ** -15
        assert np.abs(rec - dec.astype(np.float64)).max() <= (tol + 3e-7) * np.abs(dec).max()


@pytest.mark.parametrize("prec,int_path", [(0, 0), (1, 0), (2, 0), (3, 0), (4, 0), (5, 0), (3, 1), (4, 1), (5, 1)])
@pytest.mark.parametrize("out,inn,n", [(16, 256, 1), (100, 1024, 2), (1000, 8192, 3), (130, 512, 4), (257, 4096, 8),
                                       (10, 1024, 1), (128, 16384, 5), (48, 2048, 6), (33, 512, 7)])
def test_gemv_against_float64(spg, k, oracle, prec, int_path, out, inn, n):
    """Fused dequant-GEMV (all six stored precisions, both the bf16-term path and the integer-digit path of the
    integer formats, ragged row blocks) vs a float64 product of the decoded weights.  bf16 path: exact products,
    fp32 summation.  Integer path: exact sums of 28-bit fixed-point activations (scale = the row's maximum)."""
    import torch
    k.spgk_gemv_set_int_path(int_path)
    rng = np.random.default_rng(out * 31 + inn + n)
    vals = (rng.standard_normal(out * inn) / np.sqrt(inn)).astype(np.float32)
    raw = oracle.Oracle.encode(vals, prec)
    dec = oracle.Oracle.decode(raw, out * inn, prec).astype(np.float64).reshape(out, inn)
    skip = 4 if prec >= 3 else 0
    amax = float(np.frombuffer(raw[:4].tobytes(), np.float32)[0]) if skip else 1.0
    scale = amax / {3: 127.0, 4: 7.0, 5: 1.0}[prec] if skip else 1.0
    payload = torch.from_numpy(np.concatenate([raw[skip:], np.zeros(256, np.uint8)])).cuda()
    bias = rng.standard_normal(out).astype(np.float32) * 0.1
    bd = torch.from_numpy(bias).cuda()
    act = [1, 6, 3, 2, 0, 4, 5][(out + n) % 7]                 # 5 = softmax, finished by the last CTA of the kernel
    L = spg.abi.KLayer(payload.data_ptr(), bd.data_ptr(), scale, inn, out, prec, act)
    x = rng.standard_normal((n, inn)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    y = torch.full((n + 1, out), -9.0, device="cuda")
    nbytes = k.spgk_gemv_scratch_bytes(C.byref(L), n)
    if inn * {0: 32, 1: 16, 2: 16, 3: 8, 4: 4, 5: 2}[prec] // 8 < 64:
        assert nbytes == 0                    # packed rows shorter than one 64-byte step: not this kernel's case
        return
    assert nbytes > 0
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    for rep in range(2):                      # the second call checks the ticket counters were left at zero
        rc = k.spgk_layer_gemv(C.byref(L), xd.data_ptr(), inn, y.data_ptr(), out, n, scratch.data_ptr(), None)
        assert rc == 0, k.spgk_error_string()
        torch.cuda.synchronize()
        want = x.astype(np.float64) @ dec.T + bias
        if act != 5 or n == 1:                # more than one row: a softmax layer is left as logits for spgk_softmax_rows
            want = ACT[act](want)
        got = y.cpu().numpy()
        assert np.all(got[n] == -9.0)
        # bf16 path, one row: three bf16 terms (24 bits); more rows: two terms (16 bits) per activation
        tol = (3e-6 if n == 1 or int_path else 3e-5) * max(1.0, np.abs(want).max()) * np.sqrt(inn / 256)
        assert np.abs(got[:n] - want).max() <= tol, (rep, np.abs(got[:n] - want).max())
    k.spgk_gemv_set_int_path(1)


def test_gemv_declines_unaligned_rows(spg, k):
    import torch
    payload = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    bias = torch.zeros(16, device="cuda")
    L = spg.abi.KLayer(payload.data_ptr(), bias.data_ptr(), 1.0, 784, 16, 4, 1)      # 392-byte INT4 rows
    assert k.spgk_gemv_scratch_bytes(C.byref(L), 1) == 0
    x = torch.zeros(784, device="cuda")
    y = torch.zeros(16, device="cuda")
    assert k.spgk_layer_gemv(C.byref(L), x.data_ptr(), 784, y.data_ptr(), 16, 1, payload.data_ptr(), None) == -5


@pytest.mark.parametrize("prec", [2, 3, 4, 5])
@pytest.mark.parametrize("out,inn,n", [(128, 256, 1), (100, 1024, 2), (1000, 8192, 3), (130, 512, 8), (257, 4096, 16),
                                       (640, 2048, 64), (16, 16384, 5), (300, 1280, 128)])
def test_wstream_against_float64(spg, k, oracle, prec, out, inn, n):
    """Weight-streaming tcgen05 layer (in-smem dequantisation, K splits, ragged row tiles) vs a float64 product of
    the decoded weights; products are exact, so only fp32 accumulation and the 16/24-bit activation split remain."""
    import torch
    lib = k
    vp = C.c_void_p
    lib.spgk_wstream_scratch_bytes.argtypes = [C.POINTER(spg.abi.KLayer), C.c_uint32]
    lib.spgk_wstream_scratch_bytes.restype = C.c_size_t
    lib.spgk_layer_wstream.argtypes = [C.POINTER(spg.abi.KLayer), vp, vp, vp, vp, C.c_uint32, vp, C.c_uint32, C.c_uint32, vp, vp]
    lib.spgk_wstream_status.argtypes = [vp, vp]
    rng = np.random.default_rng(out * 17 + inn + n)
    vals = (rng.standard_normal(out * inn) / np.sqrt(inn)).astype(np.float32)
    raw = oracle.Oracle.encode(vals, prec)
    dec = oracle.Oracle.decode(raw, out * inn, prec).astype(np.float64).reshape(out, inn)
    skip = 4 if prec >= 3 else 0
    amax = float(np.frombuffer(raw[:4].tobytes(), np.float32)[0]) if skip else 1.0
    scale = amax / {3: 127.0, 4: 7.0, 5: 1.0}[prec] if skip else 1.0
    payload = torch.from_numpy(np.concatenate([raw[skip:], np.zeros(256, np.uint8)])).cuda()
    bias = rng.standard_normal(out).astype(np.float32) * 0.1
    bd = torch.from_numpy(bias).cuda()
    act = [1, 6, 3, 2, 0, 4][(out + n) % 6]
    L = spg.abi.KLayer(payload.data_ptr(), bd.data_ptr(), scale, inn, out, prec, act)
    x = rng.standard_normal((n, inn)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    y = torch.full((n + 1, out), -9.0, device="cuda")
    nbytes = lib.spgk_wstream_scratch_bytes(C.byref(L), n)
    assert nbytes > 0
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    for rep in range(2):                      # the second call checks the ticket counters were left at zero
        rc = lib.spgk_layer_wstream(C.byref(L), None, None, None, xd.data_ptr(), inn, y.data_ptr(), out, n, scratch.data_ptr(), None)
        assert rc == 0, lib.spgk_error_string()
        assert lib.spgk_wstream_status(scratch.data_ptr(), None) == 0, lib.spgk_error_string()
        want = ACT[act](x.astype(np.float64) @ dec.T + bias)
        got = y.cpu().numpy()
        assert np.all(got[n] == -9.0)
        tol = (3e-6 if n == 1 else 3e-5) * max(1.0, np.abs(want).max()) * np.sqrt(inn / 256)
        assert np.abs(got[:n] - want).max() <= tol, (rep, np.abs(got[:n] - want).max())


@pytest.mark.parametrize("M,N,K,H", [(256, 512, 64, 10), (1000, 1000, 512, 10), (4096, 300, 136, 16), (640, 520, 264, 3)])
@pytest.mark.parametrize("parts", [1, 2])
@pytest.mark.parametrize("hprec,hact", [(0, 5), (3, 5), (4, 1), (2, 0)])
def test_gemm_tc_with_fused_head(spg, k, oracle, M, N, K, H, parts, hprec, hact):
    """A wide layer with the narrow last layer finished in its epilogue (softmax or plain activation, head weights in
    any stored precision) vs float64 on the same rounded operands."""
    import torch
    lib = k
    vp = C.c_void_p
    lib.spgk_gemm_tc_head_supported.argtypes = [C.POINTER(spg.abi.KLayer), C.POINTER(spg.abi.KLayer)]
    lib.spgk_head_weights_bytes.argtypes = [C.POINTER(spg.abi.KLayer)]
    lib.spgk_head_weights_bytes.restype = C.c_size_t
    lib.spgk_head_weights.argtypes = [C.POINTER(spg.abi.KLayer), vp, vp]
    lib.spgk_layer_gemm_tc_head.argtypes = [C.POINTER(spg.abi.KLayer), vp, C.c_uint32, C.c_uint64, C.c_int, C.c_int,
                                            vp, C.c_uint32, C.c_uint64, C.c_int, C.c_int,
                                            C.POINTER(spg.abi.KLayer), vp, vp, C.c_uint32, C.c_uint32, vp, vp]
    rng = np.random.default_rng(M + N * 3 + K * 7 + H)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    act = [1, 3, 2, 4][(M + N) % 4]
    ld = (K + 7) & ~7
    dt = torch.bfloat16
    a16 = torch.zeros((parts, M, ld), dtype=dt, device="cuda")
    assert lib.spgk_split16(torch.from_numpy(x).cuda().data_ptr(), K, M, K, a16.data_ptr(), ld, M * ld, parts, 1, None) == 0
    w16 = torch.zeros((1, N, ld), dtype=dt, device="cuda")
    w16[0, :, :K] = torch.from_numpy(w).cuda().to(dt)
    bd = torch.from_numpy(bias).cuda()
    L = spg.abi.KLayer(w16.data_ptr(), bd.data_ptr(), 0.5, K, N, 2, act)
    # the head, stored in precision hprec
    hv = (rng.standard_normal(H * N) / np.sqrt(N)).astype(np.float32)
    raw = oracle.Oracle.encode(hv, hprec)
    hdec = oracle.Oracle.decode(raw, H * N, hprec).astype(np.float64).reshape(H, N)
    skip = 4 if hprec >= 3 else 0
    amax = float(np.frombuffer(raw[:4].tobytes(), np.float32)[0]) if skip else 1.0
    hscale = amax / {3: 127.0, 4: 7.0, 5: 1.0}[hprec] if skip else 1.0
    hpay = torch.from_numpy(np.concatenate([raw[skip:], np.zeros(256, np.uint8)])).cuda()
    hb = (rng.standard_normal(H) * 0.1).astype(np.float32)
    hbd = torch.from_numpy(hb).cuda()
    Hl = spg.abi.KLayer(hpay.data_ptr(), hbd.data_ptr(), hscale, N, H, hprec, hact)
    ok = lib.spgk_gemm_tc_head_supported(C.byref(L), C.byref(Hl))
    assert ok == (1 if N > 256 else 0)
    if not ok:
        return
    hw = torch.zeros(lib.spgk_head_weights_bytes(C.byref(Hl)) // 4, device="cuda")
    assert lib.spgk_head_weights(C.byref(Hl), hw.data_ptr(), None) == 0
    out = torch.full((M + 1, H), -7.0, device="cuda")
    st = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = lib.spgk_layer_gemm_tc_head(C.byref(L), w16.data_ptr(), ld, N * ld, 1, 1, a16.data_ptr(), ld, M * ld, parts, 1,
                                     C.byref(Hl), hw.data_ptr(), out.data_ptr(), H, M, st.data_ptr(), None)
    assert rc == 0, lib.spgk_error_string()
    assert lib.spgk_gemm_tc_status(st.data_ptr(), None) == 0
    xa = a16.float().cpu().numpy().astype(np.float64).sum(0)[:, :K]
    wa = w16.float().cpu().numpy().astype(np.float64)[0, :, :K]
    h = ACT[act](0.5 * (xa @ wa.T) + bias)
    z = h @ hdec.T + hb
    if hact == 5:
        e = np.exp(z - z.max(1, keepdims=True))
        want = e / e.sum(1, keepdims=True)
    else:
        want = ACT[hact](z)
    got = out.cpu().numpy()
    assert np.all(got[M] == -7.0)
    assert np.abs(got[:M] - want).max() <= 2e-5 * max(1.0, np.abs(want).max()), np.abs(got[:M] - want).max()


@pytest.mark.parametrize("cap,K,rows,parts", [(300, 64, [10, 20, 30, 40, 50], 2), (300, 64, [299, 7, 130], 1),
                                              (256, 784, [5, 6, 250], 2), (1000, 136, list(range(100, 240)), 2)])
def test_device_resident_row_count_with_gather_and_scatter(spg, k, cap, K, rows, parts):
    """A selection of rows known only on the device: split16 gathers them, the softmax layer runs on min(capacity, count)
    rows and scatters its output back; rows outside the selection must stay untouched (the index array beyond the
    count holds decoys)."""
    import torch
    lib = k
    vp = C.c_void_p
    lib.spgk_split16_rows.argtypes = [vp, C.c_uint32, vp, C.c_uint32, C.c_uint32, vp, C.c_uint32, C.c_uint64, C.c_int, C.c_int, vp]
    lib.spgk_set_dynamic_rows.argtypes = [vp, C.c_uint32]
    lib.spgk_set_output_rows.argtypes = [vp]
    N = 10
    rng = np.random.default_rng(cap + K)
    x = rng.standard_normal((cap, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    ld = (K + 7) & ~7
    dt = torch.bfloat16
    w16 = torch.zeros((1, N, ld), dtype=dt, device="cuda")
    w16[0, :, :K] = torch.from_numpy(w).cuda().to(dt)
    b = torch.zeros(N, device="cuda")
    L = spg.abi.KLayer(w16.data_ptr(), b.data_ptr(), 1.0, K, N, 2, 5)
    idx = (torch.arange(cap, dtype=torch.int32, device="cuda") % 97) + 150          # decoys beyond the count
    idx[:len(rows)] = torch.tensor(rows, dtype=torch.int32)
    cnt = torch.tensor([len(rows)], dtype=torch.int32, device="cuda")
    a16 = torch.zeros((parts, cap, ld), dtype=dt, device="cuda")
    out = torch.full((cap, N), -3.0, device="cuda")
    st = torch.zeros(16, dtype=torch.int32, device="cuda")
    lib.spgk_set_dynamic_rows(cnt.data_ptr(), 0)
    try:
        assert lib.spgk_split16_rows(xd.data_ptr(), K, idx.data_ptr(), cap, K, a16.data_ptr(), ld, cap * ld, parts, 1, None) == 0
        lib.spgk_set_output_rows(idx.data_ptr())
        rc = lib.spgk_layer_gemm_tc(C.byref(L), w16.data_ptr(), ld, N * ld, 1, 1, a16.data_ptr(), ld, cap * ld, parts, 1,
                                    None, 0, 0, 1, out.data_ptr(), N, cap, 1, st.data_ptr(), None)
    finally:
        lib.spgk_set_output_rows(None)
        lib.spgk_set_dynamic_rows(None, 0)
    assert rc == 0, lib.spgk_error_string()
    assert lib.spgk_gemm_tc_status(st.data_ptr(), None) == 0
    got = out.cpu().numpy()
    a = a16.float().cpu().numpy().astype(np.float64)
    assert np.all(a[:, len(rows):] == 0)                                            # the split stopped at the count
    z = a.sum(0)[:len(rows), :K] @ w16.float().cpu().numpy().astype(np.float64)[0, :, :K].T
    e = np.exp(z - z.max(1, keepdims=True))
    want = e / e.sum(1, keepdims=True)
    touched = np.where((got != -3.0).any(1))[0]
    assert touched.tolist() == sorted(rows)
    assert np.abs(got[rows] - want).max() <= 2e-6



@pytest.mark.parametrize("prec", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("count", [1, 7, 1000, (1 << 20) + 3])
def test_encode_array_matches_the_reference_bytes(spg, k, oracle, prec, count):
    """Device-side array encoder vs the oracle's restatement of write_array_compressed (itself pinned to files the
    reference wrote): byte for byte, for every precision, odd tails and awkward values."""
    import torch
    lib = k
    vp = C.c_void_p
    lib.spgk_encoded_bytes.argtypes = [C.c_uint64, C.c_int]
    lib.spgk_encoded_bytes.restype = C.c_size_t
    lib.spgk_encode_array.argtypes = [vp, C.c_uint64, C.c_int, vp, vp]
    rng = np.random.default_rng(prec * 100 + count % 97)
    x = (rng.standard_normal(count) * rng.choice([1e-3, 0.1, 1.0, 30.0])).astype(np.float32)
    special = np.array([0.0, -0.0, 1e-8, -1e-8, 6.1e-5, 65504.0, 65520.0, 1e5, -1e5, 1e-40, 0.5, -0.5, 1.5, 2.5], np.float32)
    if prec in (1, 2):                                   # the float formats also see non-finite values
        special = np.concatenate([special, np.array([np.inf, -np.inf, np.nan], np.float32)])
    m = min(count, len(special))
    x[:m] = special[:m]
    want = oracle.Oracle.encode(x, prec)
    nbytes = lib.spgk_encoded_bytes(count, prec)
    assert nbytes == len(want)
    src = torch.from_numpy(x).cuda()
    dst = torch.full((nbytes + 8,), 0xAB, dtype=torch.uint8, device="cuda")
    assert lib.spgk_encode_array(src.data_ptr(), count, prec, dst.data_ptr(), None) == 0, lib.spgk_error_string()
    got = dst.cpu().numpy()
    assert np.all(got[nbytes:] == 0xAB)
    assert np.array_equal(got[:nbytes], np.frombuffer(want.tobytes(), np.uint8))


# ---------------------------------------------------------------------------
# the three-layer MLP in one launch
# ---------------------------------------------------------------------------
def _bind_mlp3(spg, k):
    vp = C.c_void_p
    KL = C.POINTER(spg.abi.KLayer)
    k.spgk_mlp3_supported.argtypes = [KL, KL, KL, C.c_uint32]
    k.spgk_mlp3_params_bytes.argtypes = [KL, KL, KL]
    k.spgk_mlp3_params_bytes.restype = C.c_size_t
    k.spgk_mlp3_params.argtypes = [KL, KL, KL, C.c_int, vp, vp]
    k.spgk_mlp3_forward.argtypes = [KL, vp, C.c_uint32, KL, vp, C.c_uint32, KL, vp, C.c_int,
                                    vp, C.c_uint32, vp, vp, C.c_uint32, C.c_int, vp, C.c_uint32, C.c_uint32,
                                    C.c_float, vp, vp, vp, vp]


def _mlp3_case(spg, k, N, K1, N1, N2, HO, acts, t16, seed):
    """Device operands of a random three-layer net plus everything the float64 restatement needs."""
    import torch
    _bind_mlp3(spg, k)
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, K1)).astype(np.float32)
    ws = [(rng.standard_normal((o, i)) * np.sqrt(2.0 / i)).astype(np.float32) for i, o in ((K1, N1), (N1, N2), (N2, HO))]
    bs = [(rng.standard_normal(o) * 0.1).astype(np.float32) for o in (N1, N2, HO)]
    scales = [0.75, 1.25, 0.5]
    dt = torch.float16 if t16 == 0 else torch.bfloat16
    keep, layers, w16 = [], [], []
    for (w, b, s, a) in zip(ws, bs, scales, acts):
        wd, bd = torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()
        keep += [wd, bd]
        layers.append(spg.abi.KLayer(wd.data_ptr(), bd.data_ptr(), s, w.shape[1], w.shape[0], 0, a))
    for L, w in zip(layers[:2], ws[:2]):
        ld = (w.shape[1] + 7) & ~7
        t = torch.zeros((w.shape[0], ld), dtype=dt, device="cuda")
        assert k.spgk_dequant16(C.byref(L), t.data_ptr(), ld, w.shape[0] * ld, 1, t16, None) == 0, k.spgk_error_string()
        w16.append((t, ld))
    assert k.spgk_mlp3_supported(C.byref(layers[0]), C.byref(layers[1]), C.byref(layers[2]), K1) == 1
    pbytes = k.spgk_mlp3_params_bytes(C.byref(layers[0]), C.byref(layers[1]), C.byref(layers[2]))
    params = torch.zeros(pbytes // 4, dtype=torch.float32, device="cuda")
    assert k.spgk_mlp3_params(C.byref(layers[0]), C.byref(layers[1]), C.byref(layers[2]), t16, params.data_ptr(), None) == 0
    return dict(x=x, ws=ws, bs=bs, scales=scales, layers=layers, w16=w16, params=params, keep=keep, xd=torch.from_numpy(x).cuda())


def _mlp3_want(case, acts, t16, pairs):
    """float64 result from the operands the tensor cores see: one 16-bit term per value, or (pairs) the
    16-bit rounding plus the rounded remainder scaled by 2^11 (fp16) / 2^8 (bf16)."""
    lo_scale = 2048.0 if t16 == 0 else 256.0

    def operand(v):
        hi = _round16(v, t16).astype(np.float64)
        if not pairs:
            return hi
        lo = _round16(((v.astype(np.float64) - hi) * lo_scale).astype(np.float32), t16).astype(np.float64)
        return hi + lo / lo_scale
    w16 = [t.float().cpu().numpy()[:, :w.shape[1]].astype(np.float64) for (t, _), w in zip(case["w16"], case["ws"][:2])]
    s, b = case["scales"], case["bs"]
    h1 = ACT[acts[0]](operand(case["x"]) @ w16[0].T * s[0] + b[0]).astype(np.float32)
    h2 = ACT[acts[1]](operand(h1) @ w16[1].T * s[1] + b[1]).astype(np.float32)
    w3 = _round16(case["ws"][2], t16).astype(np.float64)          # the head's weights enter as a 16-bit operand as well
    z = operand(h2) @ w3.T * s[2] + b[2]
    return ACT[acts[2]](z), z


def _mlp3_run(spg, k, case, t16, N, HO, rows_idx=None, rows_limit=None, pairs=0, out=None, theta=0.0, margin=None):
    import torch
    L = case["layers"]
    if out is None:
        out = torch.full((case["x"].shape[0] + 1, HO), -3.0, dtype=torch.float32, device="cuda")
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    (w1, ld1), (w2, ld2) = case["w16"]
    rc = k.spgk_mlp3_forward(C.byref(L[0]), w1.data_ptr(), ld1, C.byref(L[1]), w2.data_ptr(), ld2, C.byref(L[2]),
                             case["params"].data_ptr(), t16, case["xd"].data_ptr(), case["x"].shape[1],
                             rows_idx.data_ptr() if rows_idx is not None else None,
                             rows_limit.data_ptr() if rows_limit is not None else None, 0, pairs,
                             out.data_ptr(), HO, N, theta,
                             margin[0].data_ptr() if margin else None, margin[1].data_ptr() if margin else None,
                             status.data_ptr(), None)
    assert rc == 0, k.spgk_error_string()
    assert k.spgk_gemm_tc_status(status.data_ptr(), None) == 0, k.spgk_error_string()
    return out


@pytest.mark.parametrize("N,K1,N1,N2,HO", [(1000, 784, 512, 1000, 10), (128, 64, 64, 64, 3), (300, 100, 256, 300, 16),
                                           (130, 784, 448, 260, 12), (5000, 20, 16, 16, 1), (257, 132, 200, 1024, 13)])
@pytest.mark.parametrize("t16", [0, 1])
@pytest.mark.parametrize("pairs", [0, 1])
def test_mlp3_fused_against_float64(spg, k, N, K1, N1, N2, HO, t16, pairs):
    """One-launch MLP vs float64 arithmetic on the same rounded operands (all rows, guard row untouched)."""
    acts = [[1, 1, 5], [3, 4, 5], [2, 0, 6], [4, 3, 2], [1, 6, 0], [6, 1, 5]][(N + K1 + N1) % 6]
    case = _mlp3_case(spg, k, N, K1, N1, N2, HO, acts, t16, seed=N + K1 + 31 * HO)
    got = _mlp3_run(spg, k, case, t16, N, HO, pairs=pairs).cpu().numpy()
    want, z = _mlp3_want(case, acts, t16, pairs)
    assert np.all(got[N] == -3.0)
    # one-term mode: a hidden activation that sits on a 16-bit rounding boundary may round the other way after fp32
    # accumulation than in the float64 restatement (one unit of 2^-11 / 2^-8 on one of up to 512 terms); the two-term
    # mode has no such boundary effect above 2^-22 / 2^-16
    eps = 2.0 ** -11 if t16 == 0 else 2.0 ** -8
    tol = (3e-5 + (0.25 * eps if not pairs else 0.02 * eps * eps * 2048)) * max(1.0, np.abs(z).max())
    assert np.abs(got[:N] - want).max() <= tol, (np.abs(got[:N] - want).max(), tol)


def test_mlp3_fused_row_list_limit_and_margin(spg, k):
    """Row list + device-resident row count (only the listed rows are touched), and the margin list of the one-term pass."""
    import torch
    N, K1, N1, N2, HO, t16 = 3000, 784, 512, 1000, 10, 0
    acts = [1, 1, 5]
    case = _mlp3_case(spg, k, N, K1, N1, N2, HO, acts, t16, seed=11)
    want1, z1 = _mlp3_want(case, acts, t16, 0)
    idx = torch.zeros(N, dtype=torch.int32, device="cuda")
    count = torch.zeros(4, dtype=torch.int32, device="cuda")
    theta = 0.05
    fast = _mlp3_run(spg, k, case, t16, N, HO, theta=theta, margin=(idx, count))
    assert np.abs(fast.cpu().numpy()[:N] - want1).max() < 2e-4      # one fp16 term: a hidden value on a rounding boundary may round the other way
    n = int(count[0].item())
    srt = np.sort(z1, axis=1)
    gap = srt[:, -1] - srt[:, -2]
    flagged = np.sort(idx.cpu().numpy()[:n])
    sure = np.nonzero(gap < theta - 2e-3)[0]
    maybe = np.nonzero(gap < theta + 2e-3)[0]
    assert set(sure) <= set(flagged) <= set(maybe) and n > 0
    # exact recomputation of just those rows, in place
    wantp, _ = _mlp3_want(case, acts, t16, 1)
    before = fast.clone()
    _mlp3_run(spg, k, case, t16, N, HO, rows_idx=idx, rows_limit=count, pairs=1, out=fast)
    after = fast.cpu().numpy()
    mask = np.zeros(N + 1, bool)
    mask[flagged] = True
    assert np.array_equal(after[~mask], before.cpu().numpy()[~mask])
    assert np.abs(after[:N][mask[:N]] - wantp[mask[:N]]).max() < 1e-5
    # the two-term rows agree with the full-precision product of the unrounded input far better than the one-term rows
    x64 = case["x"].astype(np.float64)
    w = [t.float().cpu().numpy()[:, :ww.shape[1]].astype(np.float64) for (t, _), ww in zip(case["w16"], case["ws"][:2])]
    s, b = case["scales"], case["bs"]
    h2 = np.maximum(np.maximum(x64 @ w[0].T * s[0] + b[0], 0) @ w[1].T * s[1] + b[1], 0)
    full = _softmax(h2 @ _round16(case["ws"][2], t16).astype(np.float64).T * s[2] + b[2])
    assert np.abs(after[:N][mask[:N]] - full[mask[:N]]).max() < 2e-5


# ---------------------------------------------------------------------------
# the reference-made edge tables on the device kernels
# ---------------------------------------------------------------------------
def _edge_check(got, want, x, exact_inf, of_nan=None):
    """Element-wise comparison with the reference's table: NaN where it has NaN, the same infinity, else 1e-5 relative.
    Kernels that carry activations as 16-bit terms cannot split an infinite input (inf - inf is NaN), so for +-inf inputs
    their pre-activation is NaN and they may answer what the activation makes of a NaN (of_nan: NaN itself, or 0 for
    ReLU, whose comparison `x > 0 ? x : 0` is false for NaN in the reference as well) instead of the table's value
    (exact_inf = False); they never answer any other number."""
    for g, w, xi in zip(got, want, x):
        if np.isnan(w):
            assert np.isnan(g), (xi, g, w)
        elif np.isinf(xi) and not exact_inf:
            assert np.isnan(g) or g == w or (of_nan is not None and g == of_nan), (xi, g, w)
        elif np.isinf(w):
            assert g == w, (xi, g, w)
        else:
            assert abs(g - w) <= 1e-5 * max(1.0, abs(w)) + 1e-30, (xi, g, w)


@pytest.mark.parametrize("act", [0, 1, 2, 3, 4, 6])
def test_activation_edge_table_on_every_layer_kernel(spg, k, act):
    """+-0, 1 +- 1 ulp (FOO52's knee), +-88, +-1e30, +-inf ... (tests/golden/activations.npz, written by the reference's own
    activate()) through a layer with identity weights and zero bias on each layer kernel: the general SIMT layer, the GEMV,
    the weight-streaming kernel, the tcgen05 GEMM and the one-launch MLP."""
    import torch
    g = np.load(__import__("conftest").golden("activations.npz"))
    x, want = g["x"], g["activate"][act]
    of_nan = float(__import__("oracle").Oracle.activate([np.nan], act)[0])     # Activation.c:23-38 on a NaN: 0 for ReLU, else NaN
    n, W = len(x), 64
    X = np.zeros((n, W), np.float32)
    X[:, 0] = x
    xd = torch.from_numpy(X).cuda()
    eye = np.eye(W, dtype=np.float32)
    wd, bd = torch.from_numpy(eye).cuda(), torch.zeros(W, device="cuda")
    L = spg.abi.KLayer(wd.data_ptr(), bd.data_ptr(), 1.0, W, W, 0, act)
    vp = C.c_void_p
    # 1. general SIMT layer (fp32): exact class behaviour, infinities included
    y = torch.zeros((n, W), device="cuda")
    assert k.spgk_layer_simt(C.byref(L), xd.data_ptr(), W, y.data_ptr(), W, n, None) == 0, k.spgk_error_string()
    _edge_check(y.cpu().numpy()[:, 0], want, x, exact_inf=True)
    # 2. GEMV (up to 8 rows a call)
    k.spgk_gemv_status.argtypes = [vp, vp]
    nb = k.spgk_gemv_scratch_bytes(C.byref(L), 8)
    if nb:
        scratch = torch.zeros(nb, dtype=torch.uint8, device="cuda")
        y.zero_()
        for r0 in range(0, n, 8):
            rows = min(8, n - r0)
            assert k.spgk_layer_gemv(C.byref(L), xd[r0:].data_ptr(), W, y[r0:].data_ptr(), W, rows, scratch.data_ptr(), None) == 0, k.spgk_error_string()
            assert k.spgk_gemv_status(scratch.data_ptr(), None) == 0
        _edge_check(y.cpu().numpy()[:, 0], want, x, exact_inf=False, of_nan=of_nan)
    # 3. weight streaming through the tensor core (bf16 identity weights)
    k.spgk_wstream_scratch_bytes.argtypes = [C.POINTER(spg.abi.KLayer), C.c_uint32]
    k.spgk_wstream_scratch_bytes.restype = C.c_size_t
    k.spgk_layer_wstream.argtypes = [C.POINTER(spg.abi.KLayer), vp, vp, vp, vp, C.c_uint32, vp, C.c_uint32, C.c_uint32, vp, vp]
    k.spgk_wstream_status.argtypes = [vp, vp]
    wb = torch.from_numpy(eye).to(torch.bfloat16).cuda()
    Lb = spg.abi.KLayer(wb.data_ptr(), bd.data_ptr(), 1.0, W, W, 2, act)
    nb = k.spgk_wstream_scratch_bytes(C.byref(Lb), n)
    if nb:
        scratch = torch.zeros(nb, dtype=torch.uint8, device="cuda")
        y.zero_()
        assert k.spgk_layer_wstream(C.byref(Lb), None, None, None, xd.data_ptr(), W, y.data_ptr(), W, n, scratch.data_ptr(), None) == 0, k.spgk_error_string()
        assert k.spgk_wstream_status(scratch.data_ptr(), None) == 0
        _edge_check(y.cpu().numpy()[:, 0], want, x, exact_inf=False, of_nan=of_nan)
    # 4. tcgen05 GEMM, two bf16 terms per activation
    a16 = torch.zeros((2, n, W), dtype=torch.bfloat16, device="cuda")
    assert k.spgk_split16(xd.data_ptr(), W, n, W, a16.data_ptr(), W, n * W, 2, 1, None) == 0
    w16 = torch.zeros((1, W, W), dtype=torch.bfloat16, device="cuda")
    assert k.spgk_dequant16(C.byref(L), w16.data_ptr(), W, W * W, 1, 1, None) == 0
    o32 = torch.zeros((n, W), device="cuda")
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    assert k.spgk_layer_gemm_tc(C.byref(L), w16.data_ptr(), W, W * W, 1, 1, a16.data_ptr(), W, n * W, 2, 1,
                                None, 0, 0, 1, o32.data_ptr(), W, n, 0, status.data_ptr(), None) == 0, k.spgk_error_string()
    assert k.spgk_gemm_tc_status(status.data_ptr(), None) == 0
    _edge_check(o32.cpu().numpy()[:, 0], want, x, exact_inf=False, of_nan=of_nan)
    # 5. the one-launch MLP in pair mode (two fp16 terms): the activation under test is layer 1's, layer 2 and the head
    #    pass the value on (identity weights, no activation); fp16 terms reach |x| <= 65504 only
    if act != 6:
        _bind_mlp3(spg, k)
        L1 = spg.abi.KLayer(wd.data_ptr(), bd.data_ptr(), 1.0, W, W, 0, act)
        L2 = spg.abi.KLayer(wd.data_ptr(), bd.data_ptr(), 1.0, W, W, 0, 6)
        eye16 = torch.from_numpy(np.eye(16, W, dtype=np.float32)).cuda()
        L3 = spg.abi.KLayer(eye16.data_ptr(), bd.data_ptr(), 1.0, W, 16, 0, 6)
        w16h = torch.from_numpy(eye).to(torch.float16).cuda()
        assert k.spgk_mlp3_supported(C.byref(L1), C.byref(L2), C.byref(L3), W) == 1
        params = torch.zeros(k.spgk_mlp3_params_bytes(C.byref(L1), C.byref(L2), C.byref(L3)) // 4, device="cuda")
        assert k.spgk_mlp3_params(C.byref(L1), C.byref(L2), C.byref(L3), 0, params.data_ptr(), None) == 0
        out = torch.zeros((n, 16), device="cuda")
        assert k.spgk_mlp3_forward(C.byref(L1), w16h.data_ptr(), W, C.byref(L2), w16h.data_ptr(), W, C.byref(L3), params.data_ptr(), 0,
                                   xd.data_ptr(), W, None, None, 0, 1, out.data_ptr(), 16, n, 0.0, None, None, status.data_ptr(), None) == 0, k.spgk_error_string()
        assert k.spgk_gemm_tc_status(status.data_ptr(), None) == 0
        got = out.cpu().numpy()[:, 0]
        small = np.abs(x) <= 60000
        _edge_check(got[small], want[small], x[small], exact_inf=False, of_nan=of_nan)


def test_softmax_edge_table_on_the_row_block_and_fused_kernels(spg, k):
    """Rows of tests/golden/softmax.npz (all -1e30, one +1e30, a single element, 88 / 89 / -90, 1000 wide ...) through the
    warp-per-row kernel, the CTA-per-row kernel (few rows wider than 64) and the softmax fused into the GEMM epilogue
    (identity weights), against the reference's apply_softmax outputs (Activation.c:5-21)."""
    import torch
    g = np.load(__import__("conftest").golden("softmax.npz"))
    nrows = len(g.files) // 2
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    for i in range(nrows):
        row, want = g[f"in{i}"], g[f"out{i}"]
        w = len(row)
        # many copies -> the warp-per-row kernel; one copy of a wide row -> the CTA-per-row kernel
        for copies in (70, 1):
            y = torch.from_numpy(np.tile(row, (copies, 1)).astype(np.float32)).cuda()
            assert k.spgk_softmax_rows(y.data_ptr(), w, copies, w, None) == 0, k.spgk_error_string()
            got = y.cpu().numpy()
            assert np.abs(got - want).max() <= 1e-6, (i, copies, np.abs(got - want).max())
        if w <= 256 and w >= 2:
            W = (w + 7) & ~7
            eye = np.eye(w, W, dtype=np.float32)
            wd, bd = torch.from_numpy(eye).cuda(), torch.zeros(w, device="cuda")
            L = spg.abi.KLayer(wd.data_ptr(), bd.data_ptr(), 1.0, W, w, 0, 5)
            X = np.zeros((3, W), np.float32)
            X[:, :w] = row
            xd = torch.from_numpy(X).cuda()
            a16 = torch.zeros((2, 3, W), dtype=torch.bfloat16, device="cuda")
            assert k.spgk_split16(xd.data_ptr(), W, 3, W, a16.data_ptr(), W, 3 * W, 2, 1, None) == 0
            w16 = torch.zeros((1, w, W), dtype=torch.bfloat16, device="cuda")
            assert k.spgk_dequant16(C.byref(L), w16.data_ptr(), W, w * W, 1, 1, None) == 0
            o32 = torch.zeros((3, w), device="cuda")
            assert k.spgk_layer_gemm_tc(C.byref(L), w16.data_ptr(), W, w * W, 1, 1, a16.data_ptr(), W, 3 * W, 2, 1,
                                        None, 0, 0, 1, o32.data_ptr(), w, 3, 1, status.data_ptr(), None) == 0, k.spgk_error_string()
            assert k.spgk_gemm_tc_status(status.data_ptr(), None) == 0
            got = o32.cpu().numpy()
            # the logits pass through two bf16 terms (16 significant bits): 2^-16 relative on a logit of 88 moves e^x by 1e-3
            tol = 1e-6 if np.abs(row).max() < 20 or np.abs(row).max() > 1e20 else 3e-3
            assert np.abs(got - want).max() <= tol, (i, np.abs(got - want).max())


@pytest.mark.parametrize("rows,width,K", [(8192, 1000, 64), (8300, 1024, 136), (9000, 513, 72)])
def test_wide_softmax_fused_in_the_gemm_epilogue(spg, k, rows, width, K):
    """A softmax layer wider than one 256-column tile, finished inside the GEMM kernel (the CTA owns the row tile: raw logits
    per column tile, then sum and normalisation row by row) against float64 on the same two-term operands, with the margin
    list it writes on the way; the last row tile is ragged."""
    import torch
    k.spgk_gemm_tc_softmax_fusable.argtypes = [C.c_uint32, C.c_uint32, C.c_int]
    assert k.spgk_gemm_tc_softmax_fusable(width, rows, 0) == 1
    assert k.spgk_gemm_tc_softmax_fusable(width, rows, 1) == 0 and k.spgk_gemm_tc_softmax_fusable(width, 4096, 0) == 0
    assert k.spgk_gemm_tc_softmax_fusable(200, 5, 1) == 1 and k.spgk_gemm_tc_softmax_fusable(1025, rows, 0) == 0
    rng = np.random.default_rng(rows + width)
    w = (rng.standard_normal((width, K)) * 2.0 / np.sqrt(K)).astype(np.float32)
    b = (rng.standard_normal(width) * 0.3).astype(np.float32)
    x = rng.standard_normal((rows, K)).astype(np.float32)
    ld = (K + 7) & ~7
    wd, bd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda(), torch.from_numpy(x).cuda()
    L = spg.abi.KLayer(wd.data_ptr(), bd.data_ptr(), 1.0, K, width, 0, 5)
    a16 = torch.zeros((2, rows, ld), dtype=torch.bfloat16, device="cuda")
    assert k.spgk_split16(xd.data_ptr(), K, rows, K, a16.data_ptr(), ld, rows * ld, 2, 1, None) == 0
    w16 = torch.zeros((2, width, ld), dtype=torch.bfloat16, device="cuda")
    assert k.spgk_dequant16(C.byref(L), w16.data_ptr(), ld, width * ld, 2, 1, None) == 0
    out = torch.full((rows + 1, width), -7.0, device="cuda")
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    idx = torch.zeros(rows, dtype=torch.int32, device="cuda")
    count = torch.zeros(4, dtype=torch.int32, device="cuda")
    theta = 0.02
    k.spgk_set_margin_sink.argtypes = [C.c_float, C.c_void_p, C.c_void_p]
    k.spgk_set_margin_sink(theta, idx.data_ptr(), count.data_ptr())
    try:
        rc = k.spgk_layer_gemm_tc(C.byref(L), w16.data_ptr(), ld, width * ld, 2, 1, a16.data_ptr(), ld, rows * ld, 2, 1,
                                  None, 0, 0, 1, out.data_ptr(), width, rows, 1, status.data_ptr(), None)
    finally:
        k.spgk_set_margin_sink(0.0, None, None)
    assert rc == 0, k.spgk_error_string()
    assert k.spgk_gemm_tc_status(status.data_ptr(), None) == 0, k.spgk_error_string()
    got = out.cpu().numpy()
    assert np.all(got[rows] == -7.0)                                     # nothing written past the batch
    xs = a16.float().cpu().numpy()[:, :, :K].astype(np.float64).sum(0)
    ws = w16.float().cpu().numpy()[:, :, :K].astype(np.float64).sum(0)
    z = xs @ ws.T + b.astype(np.float64)
    want = _softmax(z)
    assert np.abs(got[:rows] - want).max() <= 2e-5, np.abs(got[:rows] - want).max()      # fp32 accumulation of logits up to about 8
    assert np.allclose(got[:rows].sum(1), 1.0, atol=1e-5)
    srt = np.sort(z, axis=1)
    gap = srt[:, -1] - srt[:, -2]
    n = int(count[0].item())
    flagged = set(idx.cpu().numpy()[:n].tolist())
    assert len(flagged) == n and n > 0
    assert set(np.nonzero(gap < theta - 1e-4)[0].tolist()) <= flagged <= set(np.nonzero(gap < theta + 1e-4)[0].tolist())


def test_a_bounded_device_wait_that_runs_out_is_reported_not_hung(spg, k):
    """A barrier nobody arrives on, waited for with the tensor-core kernels' own bounded waits and a small limit: the kernel
    returns by itself, the status word carries the wait's code, the host call answers SPGK_E_TIMEOUT (which the library
    maps to SPINGALETT_ERR_DEVICE), and the context is as usable afterwards as before."""
    import torch
    k.spgk_selftest_bounded_wait.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p]
    st = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = k.spgk_selftest_bounded_wait(st.data_ptr(), 32, None)
    assert rc == -4, (rc, k.spgk_error_string())                     # SPGK_E_TIMEOUT
    assert b"bounded wait 41" in k.spgk_error_string()
    host = st.cpu().numpy()
    assert host[0] == 0 and host[1] == 0 and host[2] == 2            # word cleared by the status call; warp 1 saw the abort flag
    # the context still works: any other kernel runs
    y = torch.ones((4, 8), device="cuda")
    assert k.spgk_softmax_rows(y.data_ptr(), 8, 4, 8, None) == 0
    assert abs(float(y.sum()) - 4.0) < 1e-5


def test_injected_allocation_failures_are_reported_and_leak_nothing(spg, k):
    """The k-th device allocation fails (host-side injection): upload, batched forward and train() each answer ERR_ALLOC and
    give back what they had taken -- free device memory returns to its level."""
    import torch
    lib, a = spg.lib(), spg.abi
    lib.spgk_mem_info.argtypes = [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]

    def free_bytes():
        torch.cuda.synchronize()
        f = C.c_size_t(0)
        assert lib.spgk_mem_info(C.byref(f), None) == 0
        return f.value
    x = np.random.default_rng(0).random((2048, 20), dtype=np.float32)
    t = np.zeros((2048, 10), np.float32)
    t[:, 3] = 1.0
    # one clean pass first: the driver loads each kernel's module on first use and takes device memory for it
    warm = spg.Network.build([20, 33, 17, 10], [a.ACT_RELU, a.ACT_FOO52, a.ACT_SOFTMAX], a.WEIGHT_INITIALIZATION_HE, seed=5)
    warm.forward_batch(x)
    warm.train(x, t, epochs=1, batch_size=256)
    warm.free()
    seen_fail = 0
    for kth in range(1, 40):
        net = spg.Network.build([20, 33, 17, 10], [a.ACT_RELU, a.ACT_FOO52, a.ACT_SOFTMAX], a.WEIGHT_INITIALIZATION_HE, seed=5)
        before = free_bytes()
        lib.spgk_fail_malloc_after(kth)
        try:
            try:
                net.forward_batch(x)
                net.train(x, t, epochs=1, batch_size=256)
                worked = True
            except spg.SpingalettError as e:
                worked = False
                assert e.code == a.ERR_ALLOC, (kth, e)
                seen_fail += 1
        finally:
            lib.spgk_fail_malloc_after(0)
        if not worked:
            # a failed call must have released its own buffers; what an earlier successful call of this net holds is freed with the net
            net.free()
            assert free_bytes() >= before, (kth, before, free_bytes())
        else:
            net.free()
            break
    assert seen_fail >= 10 and worked                                  # every allocation site was hit once, then the sweep ran through


@pytest.mark.parametrize("sys_scope", [0, 1])
def test_exchange_wait_times_out_and_carries_on(spg, k, sys_scope):
    """The peer-memory exchange's wait (device and system scope flavours) on a flag that nothing sets: after its bound the
    wait reports the time-out, records its code in the status word and the thread carries on -- no hang, the context stays
    usable (a kernel launched afterwards runs)."""
    import torch
    words = torch.full((16,), 99, dtype=torch.int32, device="cuda")
    k.spgk_selftest_xchg_wait.argtypes = [C.c_void_p, C.c_uint32, C.c_int, C.c_void_p]
    assert k.spgk_selftest_xchg_wait(words.data_ptr(), 2000, sys_scope, None) == 0, k.spgk_error_string()
    torch.cuda.synchronize()
    assert words[:3].tolist() == [1, 42, 7]
    assert float((torch.ones(8, device="cuda") * 2).sum().item()) == 16.0
