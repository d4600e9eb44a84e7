"""Greedy decoding on the GPU against the CPU pipeline built from the checker (tests/cpu_decoder.py): a 2-layer decoder
with Qwen3-4B's layer dimensions (hidden 2560, 32 query / 8 key-value heads of 128, SwiGLU 9728; vocabulary cut to
32768 rows to keep the CPU side short), Q4_K projections, Q6_K embedding and lm_head, weights loaded from a .bin file.
Every operator is bit-exact against its checker, so the token streams must be IDENTICAL over 64 steps; the test also
logs the smallest top-2 logit margin seen, which says how much room an inexact path would have had."""
import os
import tempfile

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from nntrainer_b200.decoder import DecoderConfig, Qwen3Decoder  # noqa: E402
from oracle import oracle as O  # noqa: E402
from oracle.cpu_decoder import CpuDecoder, synthetic_weights, write_bin  # noqa: E402


@pytest.fixture(scope="module")
def be():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nntrainer_b200 import backend, build
    build.build()
    backend.init(0)
    return backend


_CPU_RUNS = {}


def _run(be, cfg, prompt, n_new, seed, fuse=True):
    w = synthetic_weights(cfg, seed)
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "model.bin")
        write_bin(path, cfg, w)
        gpu = Qwen3Decoder(cfg, path, fuse=fuse)
        got = gpu.generate(prompt, n_new)
        be.device_status()
        gpu_logits = gpu.b["logits"].cpu().numpy()
        gpu.close()
    key = (repr(cfg), tuple(prompt), n_new, seed)
    if key in _CPU_RUNS:  # the CPU pipeline of the same model and prompt ran for the other launch sequence already
        want, last_logits, margin = _CPU_RUNS[key]
        return got, want, gpu_logits, last_logits, margin
    cos, sin = be.rope_table(cfg.head_dim, cfg.max_seq, cfg.rope_theta)
    cpu = CpuDecoder(cfg, w, cos, sin, matmul=O.ref(fast=True) if O.ref_available() else None)
    want, pos, margin = [], 0, np.inf
    for t in prompt:
        nxt = cpu.step(t, pos)
        pos += 1
    for _ in range(n_new):
        want.append(nxt)
        top2 = np.partition(cpu.last_logits, -2)[-2:]
        margin = min(margin, float(top2[1] - top2[0]))
        nxt = cpu.step(nxt, pos)
        pos += 1
    _CPU_RUNS[key] = (want, cpu.last_logits, margin)
    return got, want, gpu_logits, cpu.last_logits, margin


@pytest.mark.parametrize("fuse", [True, False], ids=["seven_launches_per_layer", "ten_launches_per_layer"])
def test_greedy_token_stream_identical_over_64_steps(be, fuse):
    """Both launch sequences: with the residual adds and norms folded into the projections' prologues, and with every
    operator in a launch of its own."""
    cfg = DecoderConfig(n_layers=2, hidden=2560, n_heads=32, n_kv_heads=8, head_dim=128, inter=9728, vocab=32768,
                        max_seq=80)
    got, want, gl, cl, margin = _run(be, cfg, prompt=[11, 4097, 32767, 5], n_new=64, seed=0, fuse=fuse)
    print(f"smallest top-2 logit margin over 64 steps: {margin:.3e}")
    assert got == want
    assert len(set(got)) > 4, "degenerate stream: the test would not notice a wrong operator"
    assert np.array_equal(gl.view(np.uint32), cl.view(np.uint32)), "final logits differ in the last bits"


def test_sliding_window_shorter_than_the_context(be):
    cfg = DecoderConfig(n_layers=1, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, inter=768, vocab=1024, max_seq=48,
                        sliding_window=16)
    got, want, gl, cl, _ = _run(be, cfg, prompt=[1, 2, 3], n_new=40, seed=1)
    assert got == want
    assert np.array_equal(gl.view(np.uint32), cl.view(np.uint32))
