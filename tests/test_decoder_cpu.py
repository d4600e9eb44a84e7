"""The checker's decoder pipeline (oracle/cpu_decoder.py, which the GPU decoder must equal token for token) against a
decoder assembled from the reference's OWN layer classes (oracle/_ref/decoder_layers_ref: EmbeddingLayer, RMSNormLayer,
FullyConnectedLayer -> Tensor::dot -> dotQnK, ReshapedRMSNormLayer, MHACoreLayer, AdditionLayer, SwiGLULayer, compiled
unmodified, wired in the order of causal_lm.cpp, weights read from the .bin file by the reference's own reader).

With the whole-row norm summed in the order that build of the reference has (no BLAS library: a float chain), the two
give the same greedy tokens over 64 steps AND the same final logits bit for bit: every operator, the file layout and
the sampling rule are the reference's. The kernels (and the checker by default) sum the whole-row norm in the order of
the reference's per-head helper instead -- the layer's own statements have no order that holds across builds (BLAS) --
and the second test shows what that costs on a random-weight model: the first tokens agree, then a difference of a few
units in the last place crosses a rounding boundary of an activation quantizer and the streams part."""
import os
import tempfile

import numpy as np
import pytest

from nntrainer_b200 import backend as be
from nntrainer_b200.decoder import DecoderConfig
from oracle import oracle as O
from oracle.cpu_decoder import CpuDecoder, synthetic_weights, write_bin

CONFIGS = {
    "two_layers_qwen3_heads": (DecoderConfig(n_layers=2, hidden=1024, n_heads=16, n_kv_heads=4, head_dim=128, inter=3072,
                                             vocab=2048, max_seq=80), [11, 409, 2047, 5], 64, 0),
    # embedding and lm_head as the two modes of the reference's TieWordEmbedding on one tensor; a vocabulary that is not
    # a multiple of the 256-row tile (the tied tensor is [vocab][hidden], so only the hidden size has to be whole blocks)
    "tied_embeddings_vocab_1000": (DecoderConfig(n_layers=1, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, inter=768,
                                                 vocab=1000, max_seq=40, tie_word_embeddings=True), [7, 999, 0], 32, 2),
    "sliding_window_16": (DecoderConfig(n_layers=1, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, inter=768, vocab=1024,
                                        max_seq=48, sliding_window=16), [1, 2, 3], 40, 1),
}


def _both(cfg, prompt, n_new, seed, whole_row_norm):
    w = synthetic_weights(cfg, seed)
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "model.bin")
        write_bin(path, cfg, w)
        ref = O.decoder_layers_ref(cfg, path, prompt, n_new)
    if ref is None:
        pytest.skip("oracle/_ref/decoder_layers_ref not built (needs a checkout of the reference at build time)")
    cos, sin = be.rope_table(cfg.head_dim, cfg.max_seq, cfg.rope_theta)
    cpu = CpuDecoder(cfg, w, cos, sin, matmul=O.ref(fast=True) if O.ref_available() else None, whole_row_norm=whole_row_norm)
    got, pos = [], 0
    for t in prompt:
        nxt = cpu.step(t, pos)
        pos += 1
    for _ in range(n_new):
        got.append(nxt)
        nxt = cpu.step(nxt, pos)
        pos += 1
    return ref, got, cpu.last_logits


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_checker_pipeline_equals_the_references_layer_classes_token_for_token_and_bit_for_bit(name):
    cfg, prompt, n_new, seed = CONFIGS[name]
    (ref_tokens, ref_logits), got, logits = _both(cfg, prompt, n_new, seed, "layer")
    assert got == ref_tokens
    assert len(set(got)) > 4, "degenerate stream: the test would not notice a wrong operator"
    assert np.array_equal(logits.view(np.uint32), ref_logits.view(np.uint32))


def test_helper_order_of_the_whole_row_norm_agrees_at_first_then_parts_on_random_weights():
    """Not a requirement, a measurement kept honest: with the whole-row norm in the per-head helper's order (what the
    kernels do) the stream starts out equal to the layer-class decoder's; on this random-weight model it parts within
    64 tokens. The first step's logits agree to a few units in the last place."""
    cfg, prompt, n_new, seed = CONFIGS["two_layers_qwen3_heads"]
    (ref_tokens, _), got, _ = _both(cfg, prompt, n_new, seed, "helper")
    same = 0
    while same < n_new and got[same] == ref_tokens[same]:
        same += 1
    print(f"helper order: first {same} of {n_new} tokens equal to the layer-class decoder's")
    assert same >= 8
