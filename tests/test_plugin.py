"""The C++ host side of the boundary (plugin/): the run-time context plug-in loads the way the reference's Engine
loads an external context and shows the name, allocator and factory behaviour the Engine relies on; its unresolved
symbols are the framework's and nothing else; the cpu_backend-shaped functions give the CPU checker's results through
the GPU and map errors to the exception types of the CPU path."""
import os
import struct
import subprocess
import tempfile

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "plugin", "_build")


@pytest.fixture(scope="module")
def built():
    from nntrainer_b200 import build as nb_build
    from oracle import oracle as O
    nb_build.build()
    subprocess.run(["make", "-C", os.path.join(ROOT, "plugin"), f"REF={O.reference_root()}"], check=True,
                   stdout=subprocess.DEVNULL)
    return BUILD


def test_backend_library_exports_the_cpu_backend_names(built):
    out = subprocess.run(["nm", "-DC", "--defined-only", os.path.join(built, "libcuda_backend.so")],
                         capture_output=True, text=True, check=True).stdout
    for fn in ("gemm_q4_0_cuda", "gemm_q4_K_cuda", "gemm_q6_K_cuda", "quantize_row_q8_K_cuda", "quantize_row_q8_0_cuda",
               "dequantize_row_q4_K_cuda", "dequantize_row_q4_0_cuda", "dequantize_row_q6_K_cuda",
               "dequantize_row_q8_K_cuda", "dequantize_row_q8_0_cuda", "register_weight_cuda", "unregister_weight_cuda"):
        assert f"nntrainer::{fn}(" in out, fn


def test_context_plugin_loads_like_an_external_context(built):
    so, probe = os.path.join(built, "libcuda_context.so"), os.path.join(built, "context_probe")
    if not (os.path.exists(so) and os.path.exists(probe)):
        pytest.skip("plug-in not built (needs the reference's headers at build time)")
    r = subprocess.run([probe, so], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    kv = dict(line.split("=", 1) for line in r.stdout.split())
    assert kv["name"] == "gpu"                       # parseComputeEngine knows cpu / gpu / qnn only
    assert kv["mem_allocator"] != "null"             # Engine::registerContext dereferences it
    assert kv["unknown_layer_rejected"] == "1" and kv["unknown_key_rejected"] == "1"
    # unresolved symbols: the C ABI, the C/C++ runtime, and of the framework only the logger, the stock layer's
    # constructor and the base class of the allocator
    out = subprocess.run(["nm", "-DC", "--undefined-only", so], capture_output=True, text=True, check=True).stdout
    syms = [l.split(" U ", 1)[1].strip() for l in out.splitlines() if " U " in l]
    fw = sorted(s for s in syms if "@" not in s and not s.startswith("nntr_cuda_"))
    allowed = {"__nntrainer_log_print", "nntrainer::FullyConnectedLayer::FullyConnectedLayer()",
               "vtable for nntrainer::MemAllocator", "typeinfo for nntrainer::MemAllocator"}
    assert set(fw) <= allowed and set(fw[:2]) == set(sorted(allowed)[:2]), fw
    defined = subprocess.run(["nm", "-D", "--defined-only", so], capture_output=True, text=True, check=True).stdout
    assert "ml_train_context_pluggable" in defined


def test_dotqnk_hook_tool_on_synthetic_text():
    """The tool finds the function by name and its body by brace matching, wraps only calls inside it, and refuses text
    it does not understand (no such function, no call inside it, no cpu_backend include, already hooked)."""
    import sys
    sys.path.insert(0, os.path.join(ROOT, "plugin"))
    try:
        import hook_dotqnk as H
    finally:
        sys.path.pop(0)
    text = ("#include <cpu_backend.h>\n#include <other.h>\nnamespace n {\n"
            "void before() {\n  gemm_q4_K(1, 2, 3, a, 3, b, 2, c, 2);\n}\n"
            "Tensor &FloatTensor::dotQnK(Tensor const &input, Tensor &output) const {\n  switch (t) {\n  case A:\n"
            "    gemm_q4_K(M, N, K, data, K, (void *)mdata, N, rdata, N);\n    break;\n  default: {\n"
            "    gemm_q6_K(M, N, K, data, K, (void *)mdata, N, rdata, N);\n  }\n  }\n  return output;\n}\n"
            "void after() {\n  gemm_q4_0(1, 2, 3, a, 3, b, 2, c, 2);\n}\n}\n")
    hooked, n = H.hook(text)
    assert n == 2
    assert hooked.count("gemm_q4_K_cuda(M, N, K, data, K, (void *)mdata, N, rdata, N);") == 1
    assert hooked.count("gemm_q6_K_cuda(") == 1 and "gemm_q4_0_cuda(" not in hooked
    assert hooked.index("#include <cuda_backend.h>") < hooked.index("#include <other.h>")
    assert "  gemm_q4_K(1, 2, 3, a, 3, b, 2, c, 2);\n}" in hooked  # the call outside the function is untouched
    for bad in (text.replace("FloatTensor::dotQnK(", "FloatTensor::dotOther("),      # no such function
                text.replace("    gemm_q4_K(M", "    other(M").replace("    gemm_q6_K(M", "    other(M"),  # nothing to wrap
                text.replace("#include <cpu_backend.h>\n", ""),                      # nowhere to put the include
                hooked):                                                              # already hooked
        with pytest.raises(ValueError):
            H.hook(bad)


def test_dotqnk_hook_compiles_in_the_reference_and_links_to_the_backend(built):
    """plugin/hook_dotqnk.py writes the compile-time branch into a temporary copy of the reference's float_tensor.cpp;
    the copy must compile against the reference's headers with and without -DENABLE_CUDA, the CUDA build must call the
    three *_cuda functions (so the reference's argument lists type-check against cuda_backend.h) with exactly the symbols
    libcuda_backend.so defines, and the build without the macro must reference none of them."""
    import sys
    from oracle import oracle as O
    ref = O.reference_root()
    src = os.path.join(ref or "", "nntrainer", "tensor", "float_tensor.cpp")
    if not ref or not os.path.exists(src):
        pytest.skip("needs a checkout of the reference")
    sys.path.insert(0, os.path.join(ROOT, "plugin"))
    try:
        import hook_dotqnk
    finally:
        sys.path.pop(0)
    with open(src, encoding="utf-8") as f:
        original = f.read()
    hooked, wrapped = hook_dotqnk.hook(original)
    assert wrapped == 4  # Q4_K, Q6_K, and the two Q4_0 calls either side of the OpenCL branch
    # without the macro the preprocessor sees the original text: every added line sits under ENABLE_CUDA
    kept = [ln for ln in hooked.splitlines() if ln not in ("#ifdef ENABLE_CUDA", "#else", "#endif", "#include <cuda_backend.h>")
            and "_cuda(" not in ln]
    stripped = [ln for ln in original.splitlines() if ln not in ("#else", "#endif")]
    assert kept == stripped
    with pytest.raises(ValueError):
        hook_dotqnk.hook(hooked)  # applying it twice is refused
    n = os.path.join(ref, "nntrainer")
    inc = [f"-I{d}" for d in (n, f"{n}/layers", f"{n}/tensor", f"{n}/utils", f"{n}/graph", f"{n}/optimizers", f"{n}/models",
                              f"{n}/compiler", f"{n}/dataset", f"{ref}/api", f"{ref}/api/ccapi/include",
                              f"{n}/tensor/cpu_backend", f"{n}/tensor/cpu_backend/x86", f"{n}/tensor/cpu_backend/fallback",
                              f"{n}/tensor/cpu_backend/ggml_interface", os.path.join(ROOT, "plugin"))]
    with tempfile.TemporaryDirectory() as tmp:
        cpp = os.path.join(tmp, "float_tensor.cpp")
        with open(cpp, "w", encoding="utf-8") as f:
            f.write(hooked)
        wanted = {}
        for tag, extra in (("cuda", ["-DENABLE_CUDA"]), ("plain", [])):
            obj = os.path.join(tmp, f"ft_{tag}.o")
            r = subprocess.run(["/usr/bin/g++", "-std=c++17", "-O0", "-fPIC", "-c", *inc, *extra, cpp, "-o", obj],
                               capture_output=True, text=True, timeout=600)
            assert r.returncode == 0, r.stderr[-2000:]
            und = subprocess.run(["nm", "--undefined-only", obj], capture_output=True, text=True, check=True).stdout
            wanted[tag] = {ln.split()[-1] for ln in und.splitlines() if "_cuda" in ln}
    assert wanted["plain"] == set()
    assert len(wanted["cuda"]) == 3
    defined = subprocess.run(["nm", "-D", "--defined-only", os.path.join(built, "libcuda_backend.so")],
                             capture_output=True, text=True, check=True).stdout
    have = {ln.split()[-1] for ln in defined.splitlines()}
    assert wanted["cuda"] <= have, wanted["cuda"] - have


REFOUT = os.path.join(ROOT, "oracle", "_ref")
# the quantized tensor classes want N % 8 == 0 for the interleaved Q4_K form and N % 256 == 0 for Q6_K
TENSOR_DOT_CASES = [("q4_K", 1, 512, 1024), ("q4_K", 6, 136, 512), ("q4_K", 9, 64, 768), ("q4_0", 1, 64, 2880),
                    ("q4_0", 5, 64, 160), ("q6_K", 1, 256, 256), ("q6_K", 3, 256, 512)]


def _tensor_dot(exe, q, M, N, K):
    """Runs one of the drivers built from the reference's tensor sources (plugin/tensor_dot_driver.cpp) on a seeded
    case; returns (exit code, output matrix or None, the checker's result, stderr)."""
    from oracle import oracle as O
    rng = np.random.default_rng(1000 * M + N + K)
    gen = {"q4_K": O.random_q4_Kx8, "q4_0": O.random_q4_0x8, "q6_K": O.random_q6_K}[q]
    B = gen(rng, N, K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    with tempfile.TemporaryDirectory() as td:
        case, res = os.path.join(td, "case.bin"), os.path.join(td, "res.bin")
        with open(case, "wb") as f:
            f.write(struct.pack("<iIII", {"q4_0": 2, "q4_K": 12, "q6_K": 14}[q], M, N, K))
            f.write(A.tobytes())
            f.write(B.tobytes())
        r = subprocess.run([exe, case, res], capture_output=True, text=True, timeout=300)
        C = np.fromfile(res, dtype=np.float32).reshape(M, N) if r.returncode == 0 else None
    return r.returncode, C, O.port().gemm(q, A, B, N), r.stderr


@pytest.mark.parametrize("q,M,N,K", TENSOR_DOT_CASES)
def test_the_references_own_tensor_dot_equals_the_checker(built, q, M, N, K):
    """nntrainer::Tensor::dot on a quantized weight tensor, linked from the reference's unmodified tensor sources (the
    call FullyConnectedLayer makes), gives the checker's bits: the port is pinned to the reference's public tensor API,
    not only to its backend functions."""
    exe = os.path.join(REFOUT, "tensor_dot_cpu")
    if not os.path.exists(exe):
        pytest.skip("driver not built (needs a checkout of the reference at build time)")
    rc, C, want, err = _tensor_dot(exe, q, M, N, K)
    assert rc == 0, err
    assert np.array_equal(C.view(np.uint32), want.view(np.uint32))


def test_hooked_tensor_dot_without_a_device_throws_what_the_cpu_path_would(built):
    """The same driver with the ENABLE_CUDA branch in FloatTensor::dotQnK: without a CUDA device the call chain ends in
    std::runtime_error (exit code 5) raised by the backend's error mapping, never in a CPU fallback; a weight tensor the
    reference's own classes reject is still std::invalid_argument from the reference (exit code 4)."""
    torch = pytest.importorskip("torch")
    exe = os.path.join(REFOUT, "tensor_dot_cuda")
    if not os.path.exists(exe):
        pytest.skip("driver not built (needs a checkout of the reference at build time)")
    rc, _, _, err = _tensor_dot(exe, "q6_K", 3, 56, 512)  # Q6_K_Tensor wants N % 256 == 0
    assert rc == 4 and "invalid_argument" in err
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present: the no-device behaviour cannot be shown here")
    rc, C, _, err = _tensor_dot(exe, "q4_K", 1, 512, 1024)
    assert rc == 5 and C is None and "runtime_error" in err, (rc, err)


def _small_model(td, tie=False):
    from nntrainer_b200.decoder import DecoderConfig
    from oracle.cpu_decoder import synthetic_weights, write_bin
    cfg = DecoderConfig(n_layers=2, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, inter=768, vocab=1024, max_seq=48,
                        tie_word_embeddings=tie)
    path = os.path.join(td, "model.bin")
    write_bin(path, cfg, synthetic_weights(cfg, 8))  # a seed whose greedy streams visit about twenty different tokens
    return cfg, path


def test_layer_class_decoder_with_the_hook_needs_a_device(built):
    """The decoder assembled from the reference's layer classes, built with the hook: without a CUDA device its first
    projection raises (the backend's std::runtime_error), it does not quietly compute on the CPU."""
    torch = pytest.importorskip("torch")
    from oracle import oracle as O
    if not os.path.exists(os.path.join(REFOUT, "decoder_layers_cuda")):
        pytest.skip("driver not built (needs a checkout of the reference at build time)")
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present: the no-device behaviour cannot be shown here")
    with tempfile.TemporaryDirectory() as td:
        cfg, path = _small_model(td)
        with pytest.raises(RuntimeError, match="cuda|CUDA"):
            O.decoder_layers_ref(cfg, path, [1, 2, 3], 4, cuda=True)


@pytest.mark.gpu
@pytest.mark.parametrize("tie", [False, True], ids=["own_lm_head", "tied_embeddings"])
def test_layer_class_decoder_with_the_hook_generates_the_cpu_builds_tokens(built, tie):
    """The drop-in at model level: the reference's own layer classes (embedding, norms, fully connected, attention,
    SwiGLU, additions), unmodified, with only the ENABLE_CUDA branch in FloatTensor::dotQnK -- every projection and the
    lm_head run in libnntr_cuda.so through the host-pointer entry points, everything else in the reference's CPU code.
    32 greedy tokens and the final logits must equal the same program built without the hook, bit for bit."""
    torch = pytest.importorskip("torch")
    from oracle import oracle as O
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not (os.path.exists(os.path.join(REFOUT, "decoder_layers_cuda")) and os.path.exists(os.path.join(REFOUT, "decoder_layers_ref"))):
        pytest.skip("drivers not built (need a checkout of the reference at build time)")
    with tempfile.TemporaryDirectory() as td:
        cfg, path = _small_model(td, tie)
        try:
            cpu_tokens, cpu_logits = O.decoder_layers_ref(cfg, path, [5, 900, 17], 32)
            gpu_tokens, gpu_logits = O.decoder_layers_ref(cfg, path, [5, 900, 17], 32, cuda=True)
        except RuntimeError as exc:
            if "(127)" in str(exc) or "error while loading shared libraries" in str(exc):
                pytest.skip("the prebuilt drivers do not start on this machine: " + str(exc)[:200])
            raise
    assert gpu_tokens == cpu_tokens
    assert len(set(cpu_tokens)) > 10, "degenerate stream: the test would not notice a wrong projection"
    assert np.array_equal(gpu_logits.view(np.uint32), cpu_logits.view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("q,M,N,K", TENSOR_DOT_CASES)
def test_hooked_tensor_dot_runs_on_the_gpu_and_equals_the_checker(built, q, M, N, K):
    """The reference's Tensor::dot, compiled from its own sources with the hook plugin/hook_dotqnk.py writes and
    -DENABLE_CUDA, linked to libcuda_backend.so: the product comes from libnntr_cuda.so and equals the CPU result bit
    for bit (decode GEMV, and GEMM rows below the tensor-core threshold)."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    exe = os.path.join(REFOUT, "tensor_dot_cuda")
    if not os.path.exists(exe):
        pytest.skip("driver not built (needs a checkout of the reference at build time)")
    rc, C, want, err = _tensor_dot(exe, q, M, N, K)
    if rc == 127 or "error while loading shared libraries" in err:
        pytest.skip("the prebuilt driver does not start on this machine: " + err.strip()[:200])
    assert rc == 0, err
    assert np.array_equal(C.view(np.uint32), want.view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("q,M,N,K", [("q4_K", 1, 512, 1024), ("q4_K", 6, 136, 512), ("q4_0", 5, 64, 160), ("q6_K", 3, 50, 512)])
def test_backend_functions_match_the_checker_through_the_gpu(built, port, q, M, N, K):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import oracle as O
    rng = np.random.default_rng(M + N)
    gen = {"q4_K": O.random_q4_Kx8, "q4_0": O.random_q4_0x8, "q6_K": O.random_q6_K}[q]
    B = gen(rng, N, K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    with tempfile.TemporaryDirectory() as td:
        case, res = os.path.join(td, "case.bin"), os.path.join(td, "res.bin")
        with open(case, "wb") as f:
            f.write(struct.pack("<iIII", {"q4_0": 2, "q4_K": 12, "q6_K": 14}[q], M, N, K))
            f.write(A.tobytes())
            f.write(B.tobytes())
        r = subprocess.run([os.path.join(built, "backend_driver"), case, res], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stdout + r.stderr
        raw = np.fromfile(res, dtype=np.uint8)
    C = raw[:M * N * 4].view(np.float32).reshape(M, N)
    qa = raw[M * N * 4:]
    assert np.array_equal(C.view(np.uint32), port.gemm(q, A, B, N).view(np.uint32))
    want_q = port.quantize_row_q8_0(A[0]) if q == "q4_0" else port.quantize_row_q8_K(A[0])
    assert np.array_equal(qa, want_q)
