"""The device-side quantisers against the reference's quantize.py (through the committed fixture) and end to end
with the GEMM."""
import os

import numpy as np
import pytest

import fp8_quant_matmul_b200 as f
import helpers as h

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_quantisers_reproduce_the_reference_bit_for_bit():
    g = np.load(os.path.join(h.GOLDEN_DIR, "quantizer_case.npz"))
    dev = torch.device("cuda:0")
    X, W = torch.from_numpy(g["X"]).to(dev), torch.from_numpy(g["W"]).to(dev)
    A, a_s = f.quantize_rowwise(X)                       # fp8_max = 448: torch.finfo(float8_e4m3fn).max
    B, b_s = f.quantize_block(W)
    torch.cuda.synchronize()
    assert np.array_equal(a_s.cpu().numpy().view(np.uint32), g["a_scale"].view(np.uint32)), \
        int((a_s.cpu().numpy() != g["a_scale"]).sum())
    assert np.array_equal(b_s.cpu().numpy().view(np.uint32), g["b_scale"].view(np.uint32))
    # both encodings of zero are the same value (an all-zero group quantises to +0 or -0 depending on the sign of x)
    a_got, b_got = A.cpu().numpy(), B.cpu().numpy()
    assert (((a_got != g["A"]) & (((a_got | g["A"]) & 0x7F) != 0)).sum()) == 0
    assert (((b_got != g["B"]) & (((b_got | g["B"]) & 0x7F) != 0)).sum()) == 0


def test_bf16_input_and_partial_blocks():
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(3)
    W = (torch.randn(208, 384, generator=gen) * 0.5).to(torch.bfloat16)          # N = 208: second block is partial
    B, b_s = f.quantize_block(W.to(dev), fp8_max=240.0)
    torch.cuda.synchronize()
    Wf = W.float().numpy()
    Bv = f.e4m3fn_to_float(B.cpu().numpy()).reshape(384, 208).T                # [N, K]
    bs = b_s.cpu().numpy().reshape(3, 2)                                        # [kb, nb]
    assert np.abs(Bv).max() <= 240.0
    for nb in range(2):
        for kb in range(3):
            blk = Wf[nb * 128:(nb + 1) * 128, kb * 128:(kb + 1) * 128]
            want_inv = np.float32(1.0) / ((np.float32(1.0) / np.float32(np.abs(blk).max())) * np.float32(240.0))
            assert bs[kb, nb] == want_inv
            deq = Bv[nb * 128:(nb + 1) * 128, kb * 128:(kb + 1) * 128] * bs[kb, nb]
            assert np.abs(deq - blk).max() <= np.abs(blk).max() / 16 + 1e-6             # e4m3: 3 mantissa bits


def test_quantise_then_gemm_approximates_the_fp32_product():
    dev = torch.device("cuda:0")
    M, N, K = 256, 384, 1024
    gen = torch.Generator().manual_seed(5)
    X = torch.randn(M, K, generator=gen)
    W = torch.randn(N, K, generator=gen) * 0.1
    A, a_s = f.quantize_rowwise(X.to(dev))
    B, b_s = f.quantize_block(W.to(dev))
    C = f.gemm(A, B, a_s, b_s, None, M, N, K)
    f.last_device_status()
    # exact parity with the CPU checker on the quantised operands ...
    ref = h.oracle_gemm(A.cpu().numpy(), B.cpu().numpy(), a_s.cpu().numpy(), b_s.cpu().numpy(), M, N, K)
    bad, first, maxerr = h.mismatches(ref, C.view(torch.int16).cpu().numpy().view(np.uint16))
    assert bad == 0, (bad, first, maxerr)
    # ... and closeness to the unquantised product (e4m3 keeps 3 mantissa bits: both operands carry ~3 % error)
    want = (X.double() @ W.double().T).numpy()
    err = np.abs(C.float().cpu().numpy() - want)
    assert err.mean() <= 0.06 * np.abs(want).mean() + 1e-3


def test_quantiser_argument_errors():
    lib = f.lib()
    dev = torch.device("cuda:0")
    X = torch.zeros(128, 256, device=dev)
    out = torch.zeros(128 * 256, dtype=torch.uint8, device=dev)
    sc = torch.zeros(256, device=dev)
    args = (X.data_ptr(), 0, out.data_ptr(), sc.data_ptr())
    assert lib.fp8bs_quantize_rowwise(None, 0, out.data_ptr(), sc.data_ptr(), 128, 256, 448.0, None) == -1
    assert lib.fp8bs_quantize_rowwise(*args, 128, 200, 448.0, None) == -2          # K % 128
    assert lib.fp8bs_quantize_rowwise(*args, 120, 256, 448.0, None) == -3          # rows % 16
    assert lib.fp8bs_quantize_block(*args, 128, 256, 500.0, None) == -5            # beyond the e4m3fn range


def test_fnuz_bytes_from_the_reference_format_are_ingested_on_the_device():
    # operands stored as e4m3fnuz (the reference's element type, check.cu:17-21): convert on the device, run the GEMM,
    # compare with the CPU checker decoding the ORIGINAL bytes as fnuz
    dev = torch.device("cuda:0")
    M, N, K = 256, 256, 512
    A_fn, B_fn, a_s, b_s = h.make_inputs(M, N, K, seed=77)              # values common to both dialects
    to_fnuz = lambda b: np.where((b & 0x7F) == 0, 0, b + 8).astype(np.uint8)
    A_z, B_z = to_fnuz(A_fn), to_fnuz(B_fn)
    dA, nA = f.fnuz_to_fn_device(torch.from_numpy(A_z).to(dev))
    dB, nB = f.fnuz_to_fn_device(torch.from_numpy(B_z).to(dev))
    assert nA == 0 and nB == 0
    assert np.array_equal(dA.cpu().numpy(), A_fn) and np.array_equal(dB.cpu().numpy(), B_fn)
    C = f.gemm(dA, dB, torch.from_numpy(a_s).to(dev), torch.from_numpy(b_s).to(dev), None, M, N, K)
    ref = h.oracle_gemm(A_z, B_z, a_s, b_s, M, N, K, dialect=1)
    bad, first, maxerr = h.mismatches(ref, C.view(torch.int16).cpu().numpy().view(np.uint16))
    assert bad == 0, (bad, first, maxerr)
    # every byte value: agrees with the host converter where that one accepts the byte; the rest is counted
    allb = np.arange(256, dtype=np.uint8).repeat(3)[:-5]               # 763 bytes: exercises the ragged tail too
    d, inexact = f.fnuz_to_fn_device(torch.from_numpy(allb).to(dev))
    got = d.cpu().numpy()
    L = h.oracle_lib()
    n_bad = 0
    for s_, g_ in zip(allb, got):
        want = L.oracle_e4m3fnuz_to_float(int(s_))
        have = L.oracle_e4m3fn_to_float(int(g_))
        if want != want:
            assert have != have                                          # NaN -> NaN
        elif want == have:
            continue
        else:
            n_bad += 1
            assert abs(have - want) <= 2.0 ** -10                        # rounded to the neighbouring multiple of 2^-9
    assert n_bad == inexact and inexact > 0


def test_fnuz_words_mix_small_and_normal_bytes_in_every_position():
    # The device kernel works on 32-bit words with byte-parallel arithmetic: every pair of byte values side by side, at both
    # word alignments, must come out as the per-byte table says (a borrow or a carry must never reach the neighbouring byte)
    dev = torch.device("cuda:0")
    L = h.oracle_lib()
    fn_of_value = {}
    for g in range(256):
        v = L.oracle_e4m3fn_to_float(g)
        if v == v and not (g == 0x80):                                   # skip NaN and -0
            fn_of_value.setdefault(v, g)
    table = np.zeros(256, np.uint8)
    odd = np.zeros(256, np.int64)
    for b in range(256):
        v = L.oracle_e4m3fnuz_to_float(b)
        if v != v:
            table[b] = 0x7F
            continue
        if v not in fn_of_value:                                         # an odd multiple of 2^-10 below 2^-6
            odd[b] = 1
            v = round(v * 512.0) / 512.0                                 # Python rounds half to even
        table[b] = fn_of_value[v] if v != 0 else (b & 0x80)              # -2^-10 rounds to -0, which keeps its sign
    assert odd.sum() == 16                                               # eight magnitudes, two signs
    b0, b1 = np.meshgrid(np.arange(256, dtype=np.uint8), np.arange(256, dtype=np.uint8), indexing="ij")
    pairs = np.stack([b0.ravel(), b1.ravel()], axis=1).ravel()           # 131072 bytes
    for lead in (0, 1, 2, 3):
        buf = np.concatenate([np.full(lead, 0x38, np.uint8), pairs, np.full(5, 0x0B, np.uint8)])
        d, inexact = f.fnuz_to_fn_device(torch.from_numpy(buf).to(dev))
        assert np.array_equal(d.cpu().numpy(), table[buf]), "lead %d" % lead
        assert inexact == int(odd[buf].sum())
