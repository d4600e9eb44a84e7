"""TEST INFRASTRUCTURE ONLY. CPU pipeline of the Qwen3 decoder graph built from the checker's functions only (oracle/port.c GEMVs and
dequantizers, oracle/glue_port.c for everything around them): the reference's arithmetic, step by step, in the order
of Applications/CausalLM/causal_lm.cpp:174-233,566-706 and qwen3_causallm.cpp:33-110. Test infrastructure."""
import numpy as np

from nntrainer_b200.decoder import DecoderConfig, tensor_list
from oracle import oracle as O

BIG = 2 ** 31 - 1


class CpuDecoder:
    def __init__(self, cfg: DecoderConfig, weights: dict, cos, sin, matmul=None, whole_row_norm="helper"):
        """whole_row_norm: "helper" sums a row's squares in the order of the per-head helper (what the kernels do);
        "layer" in the order RMSNormLayer's own Tensor statements have in a build of the reference without BLAS."""
        self.c, self.w, self.cos, self.sin = cfg, weights, cos, sin
        self.P = O.port()
        self.row_norm = self.P.rms_norm if whole_row_norm == "helper" else self.P.rms_norm_layer
        self.mm = matmul or self.P
        self.kc = [np.zeros((cfg.max_seq, cfg.n_kv_heads, cfg.head_dim), dtype=np.uint16) for _ in range(cfg.n_layers)]
        self.vc = [np.zeros((cfg.max_seq, cfg.n_kv_heads, cfg.head_dim), dtype=np.uint16) for _ in range(cfg.n_layers)]
        self.shapes = {n: (d, N, K) for n, d, N, K in tensor_list(cfg)}
        self.last_logits = None

    def gemv(self, name, x):
        d, N, K = self.shapes[name]
        return self.mm.gemm(d, x[None, :], self.w[name], N)[0]

    def step(self, token: int, pos: int) -> int:
        c, P = self.c, self.P
        window = BIG if c.sliding_window is None else c.sliding_window
        row = 210 * (c.hidden // 256)
        x = P.dequantize_row("q6_K", self.w["embedding0"][token * row:(token + 1) * row], c.hidden)
        gqa = c.n_heads // c.n_kv_heads
        for i in range(c.n_layers):
            p = f"layer{i}_"
            n = self.row_norm(x, self.w[p + "attention_norm"], c.norm_eps)
            v = self.gemv(p + "wv", n)
            k = P.rms_norm(self.gemv(p + "wk", n), self.w[p + "k_norm"], c.norm_eps)
            q = P.rms_norm(self.gemv(p + "wq", n), self.w[p + "q_norm"], c.norm_eps)
            q = P.rotary(q, c.head_dim, self.cos[pos], self.sin[pos])
            self.kc[i][pos] = P.rotary(k, c.head_dim, self.cos[pos], self.sin[pos], to_fp16=True).reshape(c.n_kv_heads, -1)
            self.vc[i][pos] = P.rotary(v, c.head_dim, self.cos[pos], self.sin[pos], to_fp16=True,
                                       only_convert=True).reshape(c.n_kv_heads, -1)
            sc = P.compute_kcaches(q, self.kc[i], pos + 1, c.n_kv_heads, c.head_dim, gqa, window)
            pr = P.softmax_rows(sc, 0, sc.shape[0], None, True)
            a = P.compute_vcache(pos, pr, self.vc[i], c.n_kv_heads, gqa, c.head_dim, window).reshape(-1)
            h = x + self.gemv(p + "attention_out", a)
            n = self.row_norm(h, self.w[p + "ffn_norm"], c.norm_eps)
            act = P.swiglu(self.gemv(p + "ffn_up", n), self.gemv(p + "ffn_gate", n))
            x = h + self.gemv(p + "ffn_down", act)
        n = self.row_norm(x, self.w["output_norm"], c.norm_eps)
        # tied embeddings: the lm_head is the embedding tensor itself (TieWordEmbedding's second mode)
        self.last_logits = self.gemv("embedding0" if c.tie_word_embeddings else "output_of_causallm", n)
        return int(np.argmax(self.last_logits))  # first maximum, as std::max_element


def synthetic_weights(cfg: DecoderConfig, seed: int = 0) -> dict:
    rng = np.random.default_rng(seed)
    w = {}
    for name, d, N, K in tensor_list(cfg):
        if d == "f32":
            w[name] = rng.uniform(0.8, 1.2, N * K).astype(np.float32)
        elif d == "q4_K":
            w[name] = O.modellike_q4_Kx8(rng, N, K)
        else:
            w[name] = O.modellike_q6_K(rng, N, K)
    return w


def write_bin(path: str, cfg: DecoderConfig, weights: dict) -> None:
    """The file NeuralNetwork::load expects (nntrainer/models/neuralnet.cpp:690-712): tensors back to back, a 2-byte
    quantization-scheme word (QScheme::Q4_Kx8 = 3, nntrainer/tensor/quantizer.h:37) in front of every Q4_K tensor."""
    with open(path, "wb") as f:
        for name, d, _N, _K in tensor_list(cfg):
            if d == "q4_K":
                f.write(np.uint16(3).tobytes())
            f.write(weights[name].tobytes())
