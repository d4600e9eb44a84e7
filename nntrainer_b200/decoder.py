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
    rope_scaling_factor: float | None = None  # rope_scaling_type "yarn" with this factor (None: default rope)
    rope_scaling_max_position_embeddings: int = 4096


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

    def __init__(self, cfg: DecoderConfig, bin_path: str, device: str = "cuda", pdl: bool = False, fuse: bool = True):
        import torch
        self.torch, self.cfg, self.dev = torch, cfg, device
        self.fuse = fuse  # fold the residual adds and RMS norms into the prologues of the projections behind them
        self.tensors = tensor_list(cfg)
        self.w = be.BinWeights(bin_path, [(d, n, k) for _, d, n, k in self.tensors])
        self.ptr = {name: self.w.ptr[i] for i, (name, *_r) in enumerate(self.tensors)}
        self._shape = {name: (d, n, k) for name, d, n, k in self.tensors}
        self.pdl = pdl
        cos, sin = be.rope_table(cfg.head_dim, cfg.max_seq, cfg.rope_theta, yarn_factor=cfg.rope_scaling_factor,
                                 yarn_original_max_position_embeddings=cfg.rope_scaling_max_position_embeddings)
        tabs = (torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device))
        self.attn = [be.Attention(cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.max_seq, window=cfg.sliding_window,
                                  device=device, tables=tabs) for _ in range(cfg.n_layers)]
        f = lambda n: torch.empty(n, dtype=torch.float32, device=device)
        q_dim, kv_dim = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
        qkv, ug = f(q_dim + 2 * kv_dim), f(2 * cfg.inter)  # q | k | v and ffn_up | ffn_gate, each from one launch
        self.b = dict(x=f(cfg.hidden), h=f(cfg.hidden), n=f(cfg.hidden), qkv=qkv, q=qkv[:q_dim],
                      k=qkv[q_dim:q_dim + kv_dim], v=qkv[q_dim + kv_dim:], a=f(q_dim), o=f(cfg.hidden), ug=ug,
                      up=ug[:cfg.inter], gate=ug[cfg.inter:], act=f(cfg.inter), d=f(cfg.hidden), logits=f(cfg.vocab))
        self._tables()

    class _P:  # a raw device address with the data_ptr() face the backend helpers use
        def __init__(self, p):
            self.p = p

        def data_ptr(self):
            return self.p

    def _gemv(self, name, x, y):
        dtype, N, K = self._shape[name]
        be.gemv(dtype, N, K, x, self._P(self.ptr[name]), y, pdl=self.pdl)

    def _norm(self, x, name, out, width=None):
        be.rms_norm(x, self._P(self.ptr[name]), self.cfg.norm_eps, width=width, out=out, pdl=self.pdl)

    def _tables(self):
        """Device tables of weight addresses for the batched launches: per layer the q, k and v projections as row
        slices of equal height (one launch computes q | k | v into one buffer), and ffn_up | ffn_gate."""
        torch, c = self.torch, self.cfg
        kv_dim, q_dim = c.n_kv_heads * c.head_dim, c.n_heads * c.head_dim
        self._qkv_ok = c.fc_dtype == "q4_K" and q_dim % kv_dim == 0 and kv_dim % 8 == 0
        self._qkv_tab, self._ug_tab = [], []
        row_bytes = c.hidden // 256 * 144
        for i in range(c.n_layers):
            p = f"layer{i}_"
            if self._qkv_ok:
                ptrs = [self.ptr[p + "wq"] + j * kv_dim * row_bytes for j in range(q_dim // kv_dim)]
                ptrs += [self.ptr[p + "wk"], self.ptr[p + "wv"]]
                self._qkv_tab.append(torch.tensor(ptrs, dtype=torch.int64, device=self.dev))
                self._ug_tab.append(torch.tensor([self.ptr[p + "ffn_up"], self.ptr[p + "ffn_gate"]], dtype=torch.int64,
                                                 device=self.dev))
        # With ``fuse`` the q, k and v projections run as ONE 6144-row problem (its per-SM share fits in shared memory, so
        # it takes the resident-weights kernel): the file stores wv, wk, k_norm, wq, so the three tensors are packed
        # once into q | k | v order (8.8 MB per layer beside the loaded copy).
        self._qkv_packed = []
        if self.fuse and self._qkv_ok:
            for i in range(c.n_layers):
                p = f"layer{i}_"
                packed = torch.empty((q_dim + 2 * kv_dim) * row_bytes, dtype=torch.uint8, device=self.dev)
                off = 0
                for name, rows in ((p + "wq", q_dim), (p + "wk", kv_dim), (p + "wv", kv_dim)):
                    be.check(be.lib().nntr_cuda_memcpy(packed.data_ptr() + off, self.ptr[name], rows * row_bytes, 3))
                    off += rows * row_bytes
                self._qkv_packed.append(packed)

    def step(self, token_f, pos: int, pos_dev=None, out_idx=None, out_idx_f=None):
        """One decode step: ``token_f`` is a 1-element float device tensor holding the token id (the reference keeps
        ids as floats); returns (next id as int32 tensor, as float32 tensor). Logits stay in ``self.b['logits']``.
        With ``pos_dev`` (a device word) the position is read on the device, so the launches can be captured once into
        a CUDA graph and replayed for every later token.

        Launches per layer without ``fuse``: (residual add +) RMS norm; q | k | v projections (one batched launch);
        per-head norms + rotary + cache append + scores; softmax + values; attention_out; residual add + RMS norm;
        ffn_up | ffn_gate (one batched launch); SwiGLU; ffn_down -- ten. With ``fuse`` the two norms run in the
        prologues of the projections behind them and the SwiGLU in the epilogue of the up | gate launch -- seven. Every fusion keeps the bits of the
        separate operators."""
        c, b, pdl = self.cfg, self.b, self.pdl
        q_dim, kv_dim = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
        be.embedding(c.embedding_dtype, self._P(self.ptr["embedding0"]), token_f, c.vocab, c.hidden,
                     out=b["x"].view(1, -1), pdl=pdl)
        x = b["x"]
        fuse = self.fuse and self._qkv_ok
        for i in range(c.n_layers):
            p = f"layer{i}_"
            qk_norm = (self._P(self.ptr[p + "q_norm"]), self._P(self.ptr[p + "k_norm"]), c.norm_eps)
            if fuse:
                # 7 launches: (add +) norm + q|k|v; rotary + scores; softmax + values; o; add + norm + up|gate + SwiGLU; down
                g_att, g_ffn = self._P(self.ptr[p + "attention_norm"]), self._P(self.ptr[p + "ffn_norm"])
                if i == 0:
                    be.gemv_add_norm(c.fc_dtype, q_dim + 2 * kv_dim, c.hidden, x, None, None, g_att, c.norm_eps,
                                     self._qkv_packed[i], b["qkv"], pdl=pdl)
                else:  # the previous block's output x = h + ffn_down, and its norm
                    be.gemv_add_norm(c.fc_dtype, q_dim + 2 * kv_dim, c.hidden, b["h"], b["d"], x, g_att, c.norm_eps,
                                     self._qkv_packed[i], b["qkv"], pdl=pdl)
                self.attn[i].step(b["q"], b["k"], b["v"], pos, pos_dev=pos_dev, out=b["a"], pdl=pdl, qk_norm=qk_norm)
                self._gemv(p + "attention_out", b["a"], b["o"])
                be.gated_ffn_in(c.fc_dtype, c.inter, c.hidden, x, b["o"], b["h"], g_ffn, c.norm_eps,
                                self._P(self.ptr[p + "ffn_up"]), self._P(self.ptr[p + "ffn_gate"]), b["act"], pdl=pdl)
                self._gemv(p + "ffn_down", b["act"], b["d"])
                continue
            if i == 0:
                self._norm(x, p + "attention_norm", b["n"])
            else:  # the previous block's output x = h + ffn_down, and its norm
                be.add_rms_norm(b["h"], b["d"], self._P(self.ptr[p + "attention_norm"]), c.norm_eps, sum_out=x, out=b["n"],
                                pdl=pdl)
            if self._qkv_ok:
                be.gemv_batched(c.fc_dtype, kv_dim, c.hidden, b["n"], self._qkv_tab[i], q_dim // kv_dim + 2, b["qkv"],
                                pdl=pdl)
            else:
                self._gemv(p + "wv", b["n"], b["v"])
                self._gemv(p + "wk", b["n"], b["k"])
                self._gemv(p + "wq", b["n"], b["q"])
            # k_norm and q_norm (per-head RMS norms) run inside the rotary / cache-append launch
            self.attn[i].step(b["q"], b["k"], b["v"], pos, pos_dev=pos_dev, out=b["a"], pdl=pdl, qk_norm=qk_norm)
            self._gemv(p + "attention_out", b["a"], b["o"])
            be.add_rms_norm(x, b["o"], self._P(self.ptr[p + "ffn_norm"]), c.norm_eps, sum_out=b["h"], out=b["n"], pdl=pdl)
            if self._qkv_ok:
                be.gemv_batched(c.fc_dtype, c.inter, c.hidden, b["n"], self._ug_tab[i], 2, b["ug"], pdl=pdl)
            else:
                self._gemv(p + "ffn_up", b["n"], b["up"])
                self._gemv(p + "ffn_gate", b["n"], b["gate"])
            be.swiglu(b["up"], b["gate"], out=b["act"], pdl=pdl)
            self._gemv(p + "ffn_down", b["act"], b["d"])
        be.add_rms_norm(b["h"], b["d"], self._P(self.ptr["output_norm"]), c.norm_eps, sum_out=x, out=b["n"], pdl=pdl)
        head = "embedding0" if c.tie_word_embeddings else "output_of_causallm"
        self._gemv(head, b["n"], b["logits"])
        return be.argmax(b["logits"].view(1, -1), pdl=pdl, out=(out_idx, out_idx_f))

    def capture(self, start_pos: int):
        """Captures one decode step into a CUDA graph: the token id lives in ``self.tok_f`` (device float, rewritten by
        the step's own arg-max), the position in ``self.pos_dev`` (device word, advanced by the graph). Returns the
        graph; every ``replay()`` decodes one more token and leaves its id in ``self.tok`` / ``self.tok_f``."""
        torch = self.torch
        self.pos_dev = torch.full((2,), 0, dtype=torch.int32, device=self.dev)  # 8 bytes: the bump kernel adds to a u64
        self.pos_dev[0] = start_pos
        self.tok = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.tok_f = torch.zeros(1, dtype=torch.float32, device=self.dev)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.step(self.tok_f, 0, pos_dev=self.pos_dev, out_idx=self.tok, out_idx_f=self.tok_f)  # warm-up, eager
            self.pos_dev[0] = start_pos
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                self.step(self.tok_f, 0, pos_dev=self.pos_dev, out_idx=self.tok, out_idx_f=self.tok_f)
                be.check(be.lib().nntr_cuda_epoch_bump_dev(self.pos_dev.data_ptr(), be._stream()))
        torch.cuda.current_stream().wait_stream(s)
        return g

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
