"""Pins the CPU checker (oracle/port.c) before anything trusts it:
against byte fixtures produced by the reference's own code, and -- where the
reference build is present -- against that build on fresh seeded inputs."""
import numpy as np
import pytest

from oracle import oracle as O

K, N, M = 512, 16, 6


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


# ----------------------------- golden fixtures -----------------------------
def test_golden_activation_quantizers(golden, port):
    A = golden["A"]
    for m in range(M):
        assert np.array_equal(port.quantize_row_q8_K(A[m]), golden["q8_K_rows"][m])
        assert np.array_equal(port.quantize_row_q8_0(A[m]), golden["q8_0_rows"][m])
    assert np.array_equal(port.quantize_mat_q8_K_4x8(A[:4]), golden["q8_K_4x8"])
    assert np.array_equal(port.quantize_mat_q8_0_4x8(A[:4]), golden["q8_0_4x8"])


def test_golden_sign_rule_differs_only_where_expected(golden, port):
    """Row 3 has -amax before +amax: the row quantizer and the 4-row quantizer
    pick opposite scale signs there (and only there)."""
    A = golden["A"]
    for m in range(4):
        r0 = port.quantize_row_q8_K_rule(A[m], 0)
        r1 = port.quantize_row_q8_K_rule(A[m], 1)
        assert np.array_equal(r0, golden["q8_K_rows"][m])
        assert np.array_equal(r0, r1) == (m != 3)


@pytest.mark.parametrize("q,rb", [("q4_0", K // 32 * 18), ("q4_K", K // 256 * 144), ("q6_K", K // 256 * 210)])
def test_golden_dequant_and_repack(golden, port, q, rb):
    plain = golden[f"{q}_plain"]
    for r in range(N):
        assert np.array_equal(bits(port.dequantize_row(q, plain[r * rb:(r + 1) * rb], K)), bits(golden[f"{q}_dequant"][r]))
    if q != "q6_K":
        x8 = port.repack(q, plain, N, K)
        assert np.array_equal(x8, golden[f"{q}_x8"])
        assert np.array_equal(port.unpack(q, x8, N, K), plain)


def test_golden_q8_dequant(golden, port):
    assert np.array_equal(bits(port.dequantize_row("q8_K", golden["q8_K_rows"][0], K)), bits(golden["q8_K_dequant"]))
    assert np.array_equal(bits(port.dequantize_row("q8_0", golden["q8_0_rows"][0], K)), bits(golden["q8_0_dequant"]))


@pytest.mark.parametrize("q", ["q4_0", "q4_K", "q6_K"])
def test_golden_gemv_gemm_bit_exact(golden, port, q):
    B = golden[f"{q}_x8"] if q != "q6_K" else golden[f"{q}_plain"]
    A = golden["A"]
    assert np.array_equal(bits(port.gemm(q, A[:1], B, N)), bits(golden[f"{q}_gemv"]))
    assert np.array_equal(bits(port.gemm(q, A, B, N)), bits(golden[f"{q}_gemm"]))


def test_golden_quantization_error_is_sane(golden):
    """The reference's own loose bar (unittest_nntrainer_cpu_backend.cpp:182-293,
    457-515): dequantised weights near the fp32 weights, q6_K <= q4_K <= q4_0 error."""
    W = golden["W"]
    mse = {q: float(np.mean((golden[f"{q}_dequant"] - W) ** 2)) for q in ("q4_0", "q4_K", "q6_K")}
    assert mse["q6_K"] <= mse["q4_K"] <= mse["q4_0"] <= 1e-5
    ref = golden["A"] @ W.T
    for q in ("q4_0", "q4_K", "q6_K"):
        assert np.mean((golden[f"{q}_gemm"] - ref) ** 2) < 1e-2 * np.mean(ref ** 2)


# --------------------------- half-float conversion --------------------------
def test_fp16_roundtrip_all_halves(port):
    hs = np.arange(65536, dtype=np.uint16)
    want = hs.view(np.float16).astype(np.float32)
    for h in range(0, 65536, 7):
        got = np.float32(port.fp16_to_fp32(h))
        if np.isnan(want[h]):
            assert np.isnan(got)
        else:
            assert got.view(np.uint32) == want[h].view(np.uint32)
            assert port.fp32_to_fp16(float(want[h])) == h


def test_fp32_to_fp16_matches_numpy_rne(port):
    rng = np.random.default_rng(3)
    xs = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in (1e-8, 1e-6, 1e-4, 1, 300, 70000)])
    for x in xs:
        assert port.fp32_to_fp16(float(x)) == int(np.float32(x).astype(np.float16).view(np.uint16))


# ----------------------- port vs the reference build ------------------------
@pytest.mark.parametrize("q", ["q4_0", "q4_K", "q6_K"])
@pytest.mark.parametrize("Mx", [1, 2, 3, 4, 5, 9, 66])
def test_port_equals_reference_build(ref, port, q, Mx):
    rng = np.random.default_rng(1000 + Mx)
    Kx, Nx = 1024, 72
    W = (rng.standard_normal((Nx, Kx)) * 0.02).astype(np.float32)
    plain = ref.quantize_weight(q, W)
    B = ref.repack(q, plain, Nx, Kx) if q != "q6_K" else plain
    A = rng.standard_normal((Mx, Kx)).astype(np.float32)
    assert np.array_equal(bits(ref.gemm(q, A, B, Nx)), bits(port.gemm(q, A, B, Nx)))


@pytest.mark.parametrize("q,gen", [("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8), ("q6_K", O.random_q6_K)])
def test_port_equals_reference_on_random_bytes(ref, port, q, gen):
    rng = np.random.default_rng(77)
    B = gen(rng, 40, 768)
    for Mx in (1, 7):
        A = (rng.standard_normal((Mx, 768)) * 3).astype(np.float32)
        assert np.array_equal(bits(ref.gemm(q, A, B, 40)), bits(port.gemm(q, A, B, 40)))


def test_port_ldc_semantics_match_reference(ref, port):
    """GEMM rows honour ldc, the leftover M%4 rows are written with stride N
    (ggml_interface_omp.cpp:471-491) -- a quirk callers see, so the checker keeps it."""
    rng = np.random.default_rng(5)
    B = O.random_q4_Kx8(rng, 16, 512)
    for M in (8, 6, 7):  # 6 and 7: leftover rows land inside the ldc-strided rows and overwrite them
        A = rng.standard_normal((M, 512)).astype(np.float32)
        assert np.array_equal(bits(ref.gemm("q4_K", A, B, 16, ldc=24)), bits(port.gemm("q4_K", A, B, 16, ldc=24)))
    B0 = O.random_q4_0x8(rng, 16, 512)
    A = rng.standard_normal((6, 512)).astype(np.float32)
    assert np.array_equal(bits(ref.gemm("q4_0", A, B0, 16, ldc=24)), bits(port.gemm("q4_0", A, B0, 16, ldc=24)))


def test_avx512_build_gives_same_bits(ref):
    fast = O.ref(fast=True)
    if fast.path == ref.path:
        pytest.skip("host cannot run the AVX-512 build")
    rng = np.random.default_rng(9)
    A = rng.standard_normal((9, 1024)).astype(np.float32)
    for q, gen in (("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8), ("q6_K", O.random_q6_K)):
        B = gen(rng, 32, 1024)
        assert np.array_equal(bits(ref.gemm(q, A, B, 32)), bits(fast.gemm(q, A, B, 32)))
