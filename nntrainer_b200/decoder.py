"""Host-side mirror of the reference's Qwen3 decoder graph for greedy decoding, built from the device entry points of
the C ABI only (every tensor stays in HBM between operators; PyTorch provides the buffers and the stream).

Graph (Applications/CausalLM/causal_lm.cpp:174-233 constructModel, :566-612 createTransformerDecoderBlock,
qwen3_causallm.cpp:33-110 createAttention with per-head q/k norms, causal_lm.cpp:671-706 createMlp):

    embedding -> L x [ rms_norm -> wv, wk, k_norm, wq, q_norm -> mha_core -> attention_out -> add
                       -> rms_norm -> ffn_up, ffn_gate -> swiglu(ffn_up, ffn_gate) -> ffn_down -> add ]
              -> rms_norm -> lm_head -> arg-max (causal_lm.cpp:530-533)

The swiglu layer's first input (the one that goes through the sigmoid) is the layer NAMED ffn_up, the second the one
named ffn_gate (createMlp lists the inputs in that order; swiglu.cpp:55). Weights are read from a .bin file in the
order the layers request them (``tensor_list``).
"""
from __future__ import annotations

from dataclasses import dataclass

from . import backend as be


@dataclass
class DecoderConfig:
    n_layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    inter: int
    vocab: int
    max_seq: int
    rope_theta: float = 1e6
    norm_eps: float = 1e-6
    fc_dtype: str = "q4_K"
    embedding_dtype: str = "q6_K"
    lmhead_dtype: str = "q6_K"
    tie_word_embeddings: bool = False
    sliding_window: int | None = None


def tensor_list(c: DecoderConfig):
    """(name, dtype, N, K) of every weight in file order. Quantized tensors: N rows of K weights (N = output units)."""
    t = [("embedding0", c.embedding_dtype, c.vocab, c.hidden)]
    q_dim, kv_dim = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
    for i in range(c.n_layers):
        p = f"layer{i}_"
        t += [(p + "attention_norm", "f32", 1, c.hidden),
              (p + "wv", c.fc_dtype, kv_dim, c.hidden),
              (p + "wk", c.fc_dtype, kv_dim, c.hidden),
              (p + "k_norm", "f32", 1, c.head_dim),
              (p + "wq", c.fc_dtype, q_dim, c.hidden),
              (p + "q_norm", "f32", 1, c.head_dim),
              (p + "attention_out", c.fc_dtype, c.hidden, q_dim),
              (p + "ffn_norm", "f32", 1, c.hidden),
              (p + "ffn_up", c.fc_dtype, c.inter, c.hidden),
              (p + "ffn_gate", c.fc_dtype, c.inter, c.hidden),
              (p + "ffn_down", c.fc_dtype, c.hidden, c.inter)]
    t.append(("output_norm", "f32", 1, c.hidden))
    if not c.tie_word_embeddings:
        t.append(("output_of_causallm", c.lmhead_dtype, c.vocab, c.hidden))
    return t


class Qwen3Decoder:
    """Greedy decoding of a Qwen3-shaped dense decoder from a .bin file, batch 1, one token per step."""

    def __init__(self, cfg: DecoderConfig, bin_path: str, device: str = "cuda"):
        import torch
        self.torch, self.cfg, self.dev = torch, cfg, device
        self.tensors = tensor_list(cfg)
        self.w = be.BinWeights(bin_path, [(d, n, k) for _, d, n, k in self.tensors])
        self.ptr = {name: self.w.ptr[i] for i, (name, *_r) in enumerate(self.tensors)}
        cos, sin = be.rope_table(cfg.head_dim, cfg.max_seq, cfg.rope_theta)
        tabs = (torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device))
        self.attn = [be.Attention(cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.max_seq, window=cfg.sliding_window,
                                  device=device, tables=tabs) for _ in range(cfg.n_layers)]
        f = lambda n: torch.empty(n, dtype=torch.float32, device=device)
        q_dim, kv_dim = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
        self.b = dict(x=f(cfg.hidden), h=f(cfg.hidden), n=f(cfg.hidden), q=f(q_dim), k=f(kv_dim), v=f(kv_dim),
                      a=f(q_dim), o=f(cfg.hidden), up=f(cfg.inter), gate=f(cfg.inter), act=f(cfg.inter),
                      d=f(cfg.hidden), logits=f(cfg.vocab))

    class _P:  # a raw device address with the data_ptr() face the backend helpers use
        def __init__(self, p):
            self.p = p

        def data_ptr(self):
            return self.p

    def _gemv(self, name, x, y):
        _, dtype, N, K = next(t for t in self.tensors if t[0] == name)
        be.gemv(dtype, N, K, x, self._P(self.ptr[name]), y)

    def _norm(self, x, name, out, width=None):
        be.rms_norm(x, self._P(self.ptr[name]), self.cfg.norm_eps, width=width, out=out)

    def step(self, token_f, pos: int):
        """One decode step: ``token_f`` is a 1-element float device tensor holding the token id (the reference keeps
        ids as floats); returns (next id as int32 tensor, as float32 tensor). Logits stay in ``self.b['logits']``."""
        c, b = self.cfg, self.b
        be.embedding(c.embedding_dtype, self._P(self.ptr["embedding0"]), token_f, c.vocab, c.hidden,
                     out=b["x"].view(1, -1))
        x = b["x"]
        for i in range(c.n_layers):
            p = f"layer{i}_"
            self._norm(x, p + "attention_norm", b["n"])
            self._gemv(p + "wv", b["n"], b["v"])
            self._gemv(p + "wk", b["n"], b["k"])
            self._norm(b["k"], p + "k_norm", b["k"], width=c.head_dim)
            self._gemv(p + "wq", b["n"], b["q"])
            self._norm(b["q"], p + "q_norm", b["q"], width=c.head_dim)
            self.attn[i].step(b["q"], b["k"], b["v"], pos, out=b["a"])
            self._gemv(p + "attention_out", b["a"], b["o"])
            be.add(x, b["o"], out=b["h"])
            self._norm(b["h"], p + "ffn_norm", b["n"])
            self._gemv(p + "ffn_up", b["n"], b["up"])
            self._gemv(p + "ffn_gate", b["n"], b["gate"])
            be.swiglu(b["up"], b["gate"], out=b["act"])
            self._gemv(p + "ffn_down", b["act"], b["d"])
            be.add(b["h"], b["d"], out=x)
        self._norm(x, "output_norm", b["n"])
        head = "embedding0" if c.tie_word_embeddings else "output_of_causallm"
        self._gemv(head, b["n"], b["logits"])
        return be.argmax(b["logits"].view(1, -1))

    def generate(self, prompt_ids, n_new: int):
        """Feeds the prompt one token at a time, then ``n_new`` greedy tokens; returns them as a Python list."""
        torch = self.torch
        tok = torch.empty(1, dtype=torch.float32, device=self.dev)
        out, pos = [], 0
        for t in prompt_ids:
            tok.fill_(float(t))
            nxt, nxt_f = self.step(tok, pos)
            pos += 1
        for _ in range(n_new):
            out.append(int(nxt.item()))
            tok.copy_(nxt_f)
            nxt, nxt_f = self.step(tok, pos)
            pos += 1
        return out

    def close(self):
        self.w.close()
