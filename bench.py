#!/usr/bin/env python
"""bench.py -- the decode GEMV of NNTrainer's block-quantized matmul path on B200.

Workload (N = 1 GPU): BASELINE config "Single Q4_K x Q8_K decode GEMV": M=1,
K=4096, N=4096, weights N(0, 0.02^2) seed 0 quantized by the reference's Q4_K
quantizer and 8-row interleaved, activation N(0,1) quantized per call inside the
kernel. One "step" = one pass over a ring of RING distinct weight matrices
(RING x 9.4 MB > the 126 MB L2, so every launch streams its weights from HBM),
chained like decoder layers (each output is the next input) and launched with
programmatic dependent launch from one CUDA graph.

With --gpus P > 1 the projection is N-split: the global weight is
[4096*P, 4096], every rank holds a 4096-row shard (the same per-GPU work: weak
scaling) and every GEMV's epilogue stores its output slice straight into the
gathered vector of every rank (peer stores of (value, launch number) pairs over
NVLink); the next GEMV polls the numbers. No collective call on the data path.

Prints ONE JSON line (rank 0). `value` = algorithmic GB/s of the whole job with
inputs resident in HBM; `e2e` = the same metric through the host-pointer C ABI
(nntr_cuda_gemm_q4_K: host activation in, host output back, weights cached in
HBM); `roofline` = the GEMV kernel against the measured HBM peak;
`cpu_baseline` = the reference's own CPU code on this box's host cores.
`--impl reference` times only that CPU code, same config and metric.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_ROWS = 4096
K_COLS = 4096
RING = 48
WEIGHT_BYTES = N_ROWS * K_COLS // 256 * 144          # 9 437 184
ALG_BYTES = WEIGHT_BYTES + 4 * K_COLS + 4 * N_ROWS   # 9 469 952 per GEMV
FALLBACK_HBM_GBS = 6650.0
# the same string in both arms: the driver compares them
WORKLOAD = "cfg1 Q4_K x Q8_K decode GEMV M=1 K=4096 N=4096 per GPU, ring of %d matrices chained like decoder layers"
# dram__bytes_read.sum + dram__bytes_write.sum of one gemv_q4_K_resident_kernel launch on this workload (one ncu
# capture of three launches of the chained ring; the figure is per launch)
NCU_TRAFFIC_BYTES = 9_478_912


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# --------------------------------------------------------------------------
# inputs
# --------------------------------------------------------------------------
def make_base_weight():
    """cfg1 weight bytes (block_q4_Kx8) and how they were made."""
    from oracle import oracle as O
    rng = np.random.default_rng(0)
    if O.ref_available():
        R = O.ref()
        W = (rng.standard_normal((N_ROWS, K_COLS)) * 0.02).astype(np.float32)
        plain = R.quantize_weight("q4_K", W)
        return R.repack("q4_K", plain, N_ROWS, K_COLS), "N(0,0.02^2) seed 0, reference Q4_K quantizer + 8-row interleave"
    return O.random_q4_Kx8(rng, N_ROWS, K_COLS), "random block bytes (reference quantizer not built)"


def ring_host(base: np.ndarray) -> list[np.ndarray]:
    """RING distinct matrices with the statistics of the base one: row groups rotated."""
    g = base.reshape(N_ROWS // 8, -1)
    return [np.ascontiguousarray(np.roll(g, 11 * i, axis=0)).reshape(-1) for i in range(RING)]


# --------------------------------------------------------------------------
# clocks sampler
# --------------------------------------------------------------------------
class Clocks:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), [t.strip() for t in line.split(",")]))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for (t, r) in self.samples if t0 - 0.05 <= t <= t1 + 0.15 and len(r) >= 9] or \
               [r for (_, r) in self.samples if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[1]) for r in rows)
        reasons = set()
        for r in rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][2]), "reasons": sorted(reasons),
                "samples": len(rows)}


# --------------------------------------------------------------------------
# the reference's CPU path on the host cores
# --------------------------------------------------------------------------
def cpu_reference_gbps(ring: list[np.ndarray], budget_s: float, min_passes: int = 1):
    """Times ref_gemm_q4_K (M=1: quantize_row_q8_K + 4-thread GEMV, exactly the
    reference's driver) over the ring; returns (GB/s, description dict)."""
    from oracle import oracle as O
    os.environ.setdefault("OMP_WAIT_POLICY", "active")
    kind = "reference" if O.ref_available() else "port"
    lib = O.ref(fast=True) if kind == "reference" else O.port()
    x = np.random.default_rng(1).standard_normal((1, K_COLS)).astype(np.float32)
    for W in ring[:4]:
        lib.gemm("q4_K", x, W, N_ROWS)
    calls, t0 = 0, time.perf_counter()
    while True:
        for W in ring:
            lib.gemm("q4_K", x, W, N_ROWS)
        calls += len(ring)
        dt = time.perf_counter() - t0
        if dt >= budget_s and calls >= min_passes * len(ring):
            break
    gbps = calls * ALG_BYTES / dt / 1e9
    desc = {"value": round(gbps, 3), "unit": "GB/s", "cores": 4, "kind": kind,
            "sample": f"{calls} GEMV calls (M=1,N=K=4096) over a ring of {len(ring)} matrices in {dt:.1f} s; "
                      f"{os.path.basename(lib.path)}; host has {os.cpu_count()} logical cores, the reference's GEMV driver "
                      f"uses 4 OpenMP threads (ggml_interface_omp.cpp:406)"}
    return gbps, desc, dt / calls


def run_reference(args):
    """The reference's own CPU implementation on this box's host cores: same config, metric and step (one pass over
    the ring of weight matrices) as our arm. Rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    os.environ.setdefault("OMP_WAIT_POLICY", "active")
    base, how = make_base_weight()
    ring = ring_host(base)
    kind = "reference" if O.ref_available() else "port"
    lib = O.ref(fast=True) if kind == "reference" else O.port()
    x = np.random.default_rng(1).standard_normal((1, K_COLS)).astype(np.float32)

    def one_pass():
        for W in ring:
            lib.gemm("q4_K", x, W, N_ROWS)

    t_warm = time.perf_counter()
    n_warm = 0
    while n_warm < max(args.warmup, 1) or time.perf_counter() - t_warm < 1.0:  # at least a second: threads and clocks up
        one_pass()
        n_warm += 1
    # bound the whole run to about two minutes whatever --steps says
    t0 = time.perf_counter()
    one_pass()
    per_pass = time.perf_counter() - t0
    steps = max(1, min(args.steps, int(120.0 / max(per_pass, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass()
    dt = time.perf_counter() - t0
    value = steps * len(ring) * ALG_BYTES / dt / 1e9
    desc = {"value": round(value, 3), "unit": "GB/s", "cores": 4, "kind": kind,
            "sample": f"{steps} passes over a ring of {len(ring)} matrices ({steps * len(ring)} GEMV calls, M=1 N=K=4096) "
                      f"in {dt:.1f} s; {os.path.basename(lib.path)}; host has {os.cpu_count()} logical cores, the reference's "
                      f"GEMV driver uses 4 OpenMP threads (ggml_interface_omp.cpp:406)"}
    model = None
    if not args.no_model:
        try:
            model = reference_model_decode()
        except Exception as exc:  # noqa: BLE001  (a side figure: recorded, never fatal for the arm)
            model = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    moe = None
    if not args.no_moe:
        try:
            moe = reference_moe_layer_decode()
        except Exception as exc:  # noqa: BLE001
            moe = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    out = {"impl": "reference", "metric": "Q4_K GEMV HBM GB/s", "value": round(value, 3), "unit": "GB/s",
           "n_gpus": args.gpus, "steps": steps, "warmup": max(args.warmup, 1), "ms_per_step": round(dt / steps * 1e3, 3),
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u4xs8->s32, f32 scales",
           "data": "synthetic: " + how,
           "config": {"workload": WORKLOAD % len(ring),
                      "l2": "ring of %d MB exceeds the host's last-level cache" % (len(ring) * WEIGHT_BYTES // 2**20),
                      "note": "the same GEMV calls on the same ring of matrices; the CPU arm feeds every call the same "
                              "activation (chaining outputs changes nothing for its timing)"},
           "cpu_baseline": desc,
           "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "model_decode_reference": model, "moe_decode_reference": moe}
    print(json.dumps(out))


def reference_moe_layer_decode(reps=20):
    """One decode token through the reference's OWN mixture-of-experts layer class (causallm::MoELayer, run by
    oracle/moe_layer_ref.cpp) with the Qwen3-30B-A3B layer shape of our arm's moe_decode_step: hidden 2048, 128 experts of
    768, top-8, Q4_K experts (16 distinct expert weight sets cycled over the 128 to keep the case file small; the eight
    selected experts are what a call touches). Wall time per call on the host cores."""
    from oracle import oracle as O
    rng = np.random.default_rng(30)
    H, I, E, k, distinct = 2048, 768, 128, 8, 16
    x = rng.standard_normal((1, H)).astype(np.float32)
    router = (rng.standard_normal((H, E)) * 0.02).astype(np.float32)
    pool = [(O.random_q4_Kx8(rng, I, H), O.random_q4_Kx8(rng, I, H), O.random_q4_Kx8(rng, H, I)) for _ in range(distinct)]
    gate, up, down = ([pool[e % distinct][j] for e in range(E)] for j in range(3))
    r = O.moe_layer_ref(x, router, gate, up, down, k, timed_reps=reps)
    if r is None:
        return {"unavailable": "oracle/_ref/moe_layer_ref was not built (needs a checkout of the reference at build time)"}
    out, ms = r
    touched = k * 3 * I * H * 144 // 256 + H * E * 4
    return {"shape": "Qwen3-30B-A3B MoE layer, one token, the reference's own layer class", "us_per_layer": round(ms * 1e3, 1),
            "ms_per_token_48_layers": round(ms * 48, 3), "bytes_touched_per_layer": touched,
            "GB/s": round(touched / (ms * 1e-3) / 1e9, 2), "finite": bool(np.isfinite(out).all())}


def reference_model_decode(new_tokens=24):
    """Whole-model greedy decoding on the host cores by the reference's OWN layer classes (the decoder of
    oracle/decoder_layers_ref.cpp, built where a checkout of the reference was present): the Qwen3-4B shape of our arm's
    model_decode leg -- 36 layers, hidden 2560, 32 / 8 heads of 128, SwiGLU 9728, vocabulary 151936, Q4_K projections --
    with tied Q6_K embeddings, because the reference's Q6_K tensor class wants a width that is a multiple of 256 and
    151936 is not, so its own model ties the lm_head to the embedding tensor [vocab][hidden]. Synthetic weights, a short
    context (the CPU time per token is the 2.4 GB of weights, not the cache)."""
    import tempfile
    from nntrainer_b200.decoder import DecoderConfig
    from oracle import oracle as O
    from oracle.cpu_decoder import synthetic_weights, write_bin
    exe = os.path.join(os.path.dirname(os.path.abspath(O.__file__)), "_ref", "decoder_layers_ref")
    if not os.path.exists(exe):
        return {"unavailable": "oracle/_ref/decoder_layers_ref was not built (needs a checkout of the reference at build time)"}
    cfg = DecoderConfig(n_layers=36, hidden=2560, n_heads=32, n_kv_heads=8, head_dim=128, inter=9728, vocab=151936,
                        max_seq=new_tokens + 8, tie_word_embeddings=True)
    w = synthetic_weights(cfg, seed=5)
    wbytes = sum(int(a.nbytes) for a in w.values() if a.dtype == np.uint8)
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "qwen3_4b_shape_tied.bin")
        write_bin(path, cfg, w)
        del w
        tokens, _, ms = O.decoder_layers_ref(cfg, path, [11, 7, 5], new_tokens, timing=True)
    return {"shape": "Qwen3-4B decode, tied Q6_K embeddings, every layer the reference's own class", "tokens": new_tokens,
            "ms_per_token": round(ms, 3), "tok/s": round(1e3 / ms, 2), "weight_bytes_per_token": wbytes,
            "GB/s": round(wbytes / (ms * 1e-3) / 1e9, 2), "host_logical_cores": os.cpu_count(),
            "distinct_tokens": len(set(tokens))}


# --------------------------------------------------------------------------
# other decode GEMV shapes of the path (reported beside the headline, same method)
# --------------------------------------------------------------------------
OTHER_SHAPES = [  # (label, qtype, N, K)
    ("Qwen3-4B gate+up", "q4_K", 19456, 2560),
    ("Qwen3-4B down", "q4_K", 2560, 9728),
    ("Qwen3-4B lm_head", "q6_K", 151936, 2560),
    ("Q4_0 FFN 24576x4096", "q4_0", 24576, 4096),
]


def other_shapes(be, torch, dev, peak, steps=20):
    """Each shape: random block bytes (throughput does not depend on the values), enough distinct matrices to exceed L2,
    launches back to back from one CUDA graph with programmatic dependent launch; CUDA events on the launching stream."""
    from oracle import oracle as O
    gens = {"q4_K": O.random_q4_Kx8, "q4_0": O.random_q4_0x8, "q6_K": O.random_q6_K}
    per_w = {"q4_K": 144 / 256, "q4_0": 18 / 32, "q6_K": 210 / 256}
    out = []
    rng = np.random.default_rng(7)
    for label, q, N, K in OTHER_SHAPES:
        wbytes = int(N * K * per_w[q])
        alg = wbytes + 4 * K + 4 * N
        n_mat = max(2, min(48, int(300e6 // wbytes) + 1))
        base = torch.from_numpy(gens[q](rng, N, K)).to(dev)
        mats = [base] + [torch.roll(base, 4099 * 16 * (i + 1)) for i in range(n_mat - 1)]  # distinct memory, same statistics
        x = torch.randn(K, device=dev)
        y = torch.zeros(N, device=dev)
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            for W in mats:
                be.gemv(q, N, K, x, W, y, pdl=True)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for W in mats:
                    be.gemv(q, N, K, x, W, y, pdl=True)
            for _ in range(3):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (steps * n_mat)
        gbs = alg / (us * 1e-6) / 1e9
        out.append({"shape": label, "qtype": q, "N": N, "K": K, "us_per_launch": round(us, 3), "GB/s": round(gbs, 1),
                    "frac_of_hbm_peak": round(gbs / peak, 4), "algorithmic_bytes": alg, "distinct_matrices": n_mat})
        del mats, base
        torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------
# one decode token through all projections of a Qwen3-4B-shaped decoder (weights only: the quantized matmul path)
# --------------------------------------------------------------------------
QWEN3_4B = {"layers": 36, "hidden": 2560, "q_dim": 4096, "kv_dim": 1024, "inter": 9728, "vocab": 151936}


def decode_step_qwen3_4b(be, torch, dev, peak, steps=10):
    """Per layer four Q4_K GEMVs (fused q|k|v 6144x2560, o 2560x4096, fused gate|up 19456x2560, down 2560x9728), then
    the Q6_K lm_head 151936x2560: 145 launches, 2.36 GB of distinct weights, one CUDA graph with programmatic dependent
    launch, launches ordered like the layers of a decoder. Attention, norms and sampling are outside the quantized
    matmul path and are not run; tok/s is therefore the ceiling this path allows, not a whole-model figure. Every GEMV
    reads a fixed random activation of its input size, so values stay finite with random weights."""
    from oracle import oracle as O
    c = QWEN3_4B
    shapes = [(c["q_dim"] + 2 * c["kv_dim"], c["hidden"]), (c["hidden"], c["q_dim"]), (2 * c["inter"], c["hidden"]),
              (c["hidden"], c["inter"])]
    rng = np.random.default_rng(21)
    bases = [torch.from_numpy(O.random_q4_Kx8(rng, N, K)).to(dev) for N, K in shapes]
    layers = [[torch.roll(b, 1152 * (7 * l + 3)) if l else b for b in bases] for l in range(c["layers"])]  # whole blocks
    head = torch.from_numpy(O.random_q6_K(rng, c["vocab"], c["hidden"])).to(dev)
    xs = {K: torch.randn(K, device=dev) for K in {k for _, k in shapes}}
    ys = [torch.zeros(N, device=dev) for N, _ in shapes]
    logits = torch.zeros(c["vocab"], device=dev)
    wbytes = c["layers"] * sum(int(N * K * 144 / 256) for N, K in shapes) + c["vocab"] * (c["hidden"] // 256) * 210

    def one_token():
        for l in range(c["layers"]):
            for (N, K), W, y in zip(shapes, layers[l], ys):
                be.gemv("q4_K", N, K, xs[K], W, y, pdl=True)
        be.gemv("q6_K", c["vocab"], c["hidden"], xs[c["hidden"]], head, logits, pdl=True)

    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        one_token()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            one_token()
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
    be.device_status()
    ms = e0.elapsed_time(e1) / steps
    finite = bool(torch.isfinite(logits).all().item())
    out = {"shape": "Qwen3-4B decode, projections + lm_head (attention/norms not run)", "launches_per_token": 4 * c["layers"] + 1,
           "weight_bytes_per_token": wbytes, "ms_per_token": round(ms, 4), "tok/s": round(1e3 / ms, 1),
           "GB/s": round(wbytes / (ms * 1e-3) / 1e9, 1), "frac_of_hbm_peak": round(wbytes / (ms * 1e-3) / 1e9 / peak, 4),
           "ceiling_tok/s_at_hbm_peak": round(peak * 1e9 / wbytes, 1), "outputs_finite": finite}
    del layers, bases, head
    torch.cuda.empty_cache()
    return out


def decode_step_sharded(be, torch, dev, dist, world, rank, peak, steps=10):
    """The same four projections per layer, every one sharded by rows over the ranks (N-split, strong scaling: the model
    is fixed, a rank holds 1/world of every matrix) and chained for real: a launch reads the WHOLE gathered vector of
    the launch before it (the first K elements where the graph would have attention or the activation in between) and
    stores its row slice into every rank's gathered vector. 144 launches per token, no lm_head. Weights: N(0, 1/K)
    through the reference's quantizer where it was built (magnitudes stay level along the chain), rolled per layer.
    The last gathered vector is compared bit for bit with the same chain run on one GPU over the whole matrices."""
    from nntrainer_b200.nsplit import NSplitGroup
    from oracle import oracle as O
    c = QWEN3_4B
    shapes = [(c["q_dim"] + 2 * c["kv_dim"], c["hidden"]), (c["hidden"], c["q_dim"]), (2 * c["inter"], c["hidden"]),
              (c["hidden"], c["inter"])]
    if any((N // 8) % world for N, _ in shapes):
        return {"error": f"row groups do not divide over {world} ranks"}
    rng = np.random.default_rng(33)
    bases = []
    for N, K in shapes:
        if O.ref_available():
            R = O.ref()
            W = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
            bases.append(torch.from_numpy(R.repack("q4_K", R.quantize_weight("q4_K", W), N, K)).to(dev))
        else:
            bases.append(torch.from_numpy(O.modellike_q4_Kx8(rng, N, K)).to(dev))
    rolled = lambda l, j: torch.roll(bases[j], 1152 * (7 * l + 3)) if l else bases[j]
    nl = [N // world for N, _ in shapes]
    shard_bytes = [n * K // 256 * 144 for n, (_, K) in zip(nl, shapes)]
    shards = [[rolled(l, j)[rank * shard_bytes[j]:(rank + 1) * shard_bytes[j]].clone() for j in range(4)]
              for l in range(c["layers"])]
    n_launch = 4 * c["layers"]

    # Two gathered buffers (the streaming kernel's exchange): its "done reading" count is per launch, so launches of
    # different sizes may follow one another. The ring-of-four form keeps one slot per CTA and needs every launch of the
    # sequence to run the same number of CTAs, which these four shapes do not.
    ring = 2
    group = NSplitGroup(max(nl), n_launch, ring=ring)
    # a stalled exchange must end this leg in seconds, not minutes: 262144 polls per wait (tens of milliseconds) instead
    # of millions (a wait that runs out raises the device status, and the leg is reported as failed)
    be.check(be.lib().nntr_cuda_set_exchange_poll_limit(1 << 18))
    try:
        return _sharded_body(be, torch, dev, dist, world, rank, peak, steps, c, shapes, nl, shards, rolled, group, ring,
                             n_launch)
    finally:
        be.lib().nntr_cuda_set_exchange_poll_limit(0)  # back to the built-in limits
        group.close()
        del shards, bases
        torch.cuda.empty_cache()


def _sharded_body(be, torch, dev, dist, world, rank, peak, steps, c, shapes, nl, shards, rolled, group, ring, n_launch):
    x0 = torch.randn(c["hidden"], device=dev, generator=torch.Generator(device=dev).manual_seed(7))
    stream = torch.cuda.Stream(device=dev)

    def one_token():
        group.bump_epoch(stream.cuda_stream)
        for l in range(c["layers"]):
            for j, (N, K) in enumerate(shapes):
                i = 4 * l + j
                group.gemv("q4_K", K, x0.data_ptr() if i == 0 else group.gathered_ptr(i - 1), shards[l][j].data_ptr(), i,
                           stream.cuda_stream, pdl=True, x_tagged=i > 0, n_local=nl[j])

    barrier = dist.barrier if world > 1 else (lambda: None)

    def agree_clean(where):
        """A stalled exchange shows up as a device status on SOME ranks: agree on it, so that either every rank goes on
        or every rank raises (a rank that left alone would leave the others in a barrier it never reaches)."""
        bad = torch.tensor([1.0 if be.lib().nntr_cuda_device_status() != 0 else 0.0], device=dev)
        if world > 1:
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if float(bad.item()) != 0.0:
            be.lib().nntr_cuda_clear_device_status()
            raise RuntimeError(f"the exchange stalled in {where} (a bounded wait ran out on some rank)")

    def timed(fn):
        barrier()  # every rank has its weights: nobody waits on a peer that is still setting up
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            agree_clean("the first pass")
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn()
            for _ in range(3):
                g.replay()
            stream.synchronize()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
            agree_clean("the timed passes")
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms = timed(one_token)
    plain_ms = None
    if world == 1:  # the same chain without the exchange: plain launches, outputs in ordinary vectors
        ys = [torch.empty(N, device=dev) for N, _ in shapes]

        def plain_token():
            x = x0
            for l in range(c["layers"]):
                for j, (N, K) in enumerate(shapes):
                    be.gemv("q4_K", N, K, x, shards[l][j], ys[j], pdl=True)
                    x = ys[j]
        plain_ms = timed(plain_token)
    got = group.gathered_numpy(n_launch - 1, nl[3])
    # the same chain on this GPU alone, whole matrices
    x = x0.clone()
    for l in range(c["layers"]):
        for j, (N, K) in enumerate(shapes):
            y = torch.empty(N, device=dev)
            be.gemv("q4_K", N, K, x[:K].contiguous(), rolled(l, j), y)
            x = y
    want = x.cpu().numpy()
    ok = torch.tensor([0.0 if np.array_equal(got.view(np.uint32), want.view(np.uint32)) else 1.0], device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MAX)
    wbytes = c["layers"] * sum(int(N * K * 144 / 256) for N, K in shapes)
    out = {"shape": "Qwen3-4B decode, the four projections of every layer sharded by rows over the ranks (no lm_head)",
           "ranks": world, "gathered_buffers": ring, "launches_per_token": n_launch, "weight_bytes_per_token": wbytes,
           "plain_chain_ms_per_token": round(plain_ms, 4) if plain_ms is not None else None,
           "ms_per_token": round(ms, 4), "tok/s": round(1e3 / ms, 1), "GB/s": round(wbytes / (ms * 1e-3) / 1e9, 1),
           "frac_of_aggregate_hbm_peak": round(wbytes / (ms * 1e-3) / 1e9 / (peak * world), 4),
           "equals_single_gpu_chain": float(ok.item()) == 0.0, "finite": bool(np.isfinite(want).all()),
           "rms_of_last_vector": float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))}
    return out


# --------------------------------------------------------------------------
# whole-model greedy decoding of a Qwen3-4B-shaped decoder: every operator of the graph, weights from a .bin file
# --------------------------------------------------------------------------
def model_decode_qwen3_4b(be, torch, dev, peak, context=512, new_tokens=64, cpu_tokens=3):
    """cfg3: 36 layers, hidden 2560, 32 query / 8 key-value heads of 128, SwiGLU 9728, vocabulary 151936; Q4_K
    projections, Q6_K embedding and lm_head, fp16 key/value cache. Random block bytes scaled like N(0, 0.02^2) weights
    are written to a .bin file in the reference's layout and loaded through the library's loader. The first
    `context` cache rows are filled with random fp16 values in place of a prefill (multi-token attention is not built),
    then `new_tokens` greedy steps run from one captured CUDA graph (position and token id live on the device), every
    operator included: embedding row, RMS norms and residual adds (in the prologues of the projections behind them),
    q/k/v/o and FFN projections, per-head q/k norms, rotary embedding, attention over the cache, SwiGLU, lm_head,
    arg-max. The reference's CPU pipeline (the checker's
    functions, GEMVs from the reference's own code where it was built) decodes a few tokens of the same model beside
    it as a reported baseline."""
    import os
    import tempfile
    import time
    from nntrainer_b200.decoder import DecoderConfig, Qwen3Decoder, tensor_list
    from oracle import oracle as O
    from oracle.cpu_decoder import CpuDecoder, synthetic_weights, write_bin
    cfg = DecoderConfig(n_layers=36, hidden=2560, n_heads=32, n_kv_heads=8, head_dim=128, inter=9728, vocab=151936,
                        max_seq=context + new_tokens + 8)
    w = synthetic_weights(cfg, seed=5)
    wbytes = sum(int(a.nbytes) for n, a in w.items() if a.dtype == np.uint8)
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "qwen3_4b_shape.bin")
        write_bin(path, cfg, w)
        t0 = time.perf_counter()
        dec = Qwen3Decoder(cfg, path, pdl=True)
        load_s = time.perf_counter() - t0
    g = torch.Generator(device=dev)
    g.manual_seed(9)
    kv = []
    for a in dec.attn:
        kc = (torch.randn((context, cfg.n_kv_heads, cfg.head_dim), device=dev, generator=g) * 0.5).to(torch.float16)
        vc = (torch.randn((context, cfg.n_kv_heads, cfg.head_dim), device=dev, generator=g) * 0.5).to(torch.float16)
        a.kcache[:context].copy_(kc)
        a.vcache[:context].copy_(vc)
        kv.append((kc, vc))
    graph = dec.capture(context)
    dec.tok_f.fill_(11.0)
    stream = torch.cuda.current_stream()
    for _ in range(3):
        graph.replay()
    dec.pos_dev[0] = context  # the warm-up replays advanced the position
    dec.tok_f.fill_(11.0)
    toks = torch.zeros(new_tokens, dtype=torch.int32, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(new_tokens):
        graph.replay()
        toks[i:i + 1].copy_(dec.tok, non_blocking=True)
    e1.record(stream)
    torch.cuda.synchronize()
    be.device_status()
    ms = e0.elapsed_time(e1) / new_tokens
    got = toks.cpu().numpy().tolist()
    kv_bytes = 2 * cfg.n_layers * (context + new_tokens // 2) * cfg.n_kv_heads * cfg.head_dim * 2
    # CPU pipeline on the same model and cache, a few tokens: the token stream must be the same
    cos, sin = be.rope_table(cfg.head_dim, cfg.max_seq, cfg.rope_theta)
    cpu = CpuDecoder(cfg, w, cos, sin, matmul=O.ref(fast=True) if O.ref_available() else None)
    for i, (kc, vc) in enumerate(kv):
        cpu.kc[i][:context] = kc.cpu().numpy().view(np.uint16)
        cpu.vc[i][:context] = vc.cpu().numpy().view(np.uint16)
    t0 = time.perf_counter()
    want, nxt = [], 11
    for i in range(cpu_tokens):
        nxt = cpu.step(nxt, context + i)
        want.append(nxt)
    cpu_s = (time.perf_counter() - t0) / cpu_tokens
    n_launch = 1 + cfg.n_layers * 7 + 3 + 1  # embedding, 7 per layer, final norm + lm_head + arg-max, position bump
    out = {"shape": "Qwen3-4B-shaped decoder, whole model, batch 1, greedy, context %d" % context,
           "tokens": new_tokens, "ms_per_token": round(ms, 4), "tok/s": round(1e3 / ms, 1),
           "launches_per_token": n_launch, "weight_bytes_per_token": wbytes, "kv_cache_bytes_per_token": kv_bytes,
           "GB/s": round((wbytes + kv_bytes) / (ms * 1e-3) / 1e9, 1),
           "frac_of_hbm_peak": round((wbytes + kv_bytes) / (ms * 1e-3) / 1e9 / peak, 4),
           "bin_load_s": round(load_s, 2),
           "cpu_pipeline": {"tok/s": round(1.0 / cpu_s, 2), "tokens": cpu_tokens,
                            "gemv": "oracle/_ref (reference code, its OpenMP threading)" if O.ref_available() else "C restatement, 1 thread"},
           "first_tokens_equal_cpu": got[:cpu_tokens] == want, "distinct_tokens": len(set(got))}
    dec.close()
    del dec, kv, w
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------
# one decode token through the MoE layers of a Qwen3-30B-A3B-shaped decoder, expert-parallel over the ranks
# --------------------------------------------------------------------------
QWEN3_30B_A3B = {"layers": 48, "hidden": 2048, "experts": 128, "top_k": 8, "inter": 768}


def moe_decode_step(be, torch, dev, world, rank, steps=10):
    """48 MoE layers (router fp32 [2048,128], top-8 of 128 Q4_K experts with intermediate 768), batch 1: every layer's
    output is the next layer's input. With more than one rank the experts are split evenly (expert parallelism, the
    owners' down projections store their outputs into every rank's buffer; no collective call). Expert weights: 16
    distinct sets per projection rotated into distinct device memory for every (layer, expert) this rank owns --
    340 MB per layer in total, so L2 cannot serve a layer. Attention is outside the path and not run."""
    from oracle import oracle as O
    from nntrainer_b200 import nsplit
    c = QWEN3_30B_A3B
    H, I, E, k, Lc = c["hidden"], c["inter"], c["experts"], c["top_k"], c["layers"]
    rng = np.random.default_rng(31)
    pool = [[torch.from_numpy(O.random_q4_Kx8(rng, n, kk)).to(dev) for _ in range(16)] for n, kk in ((I, H), (I, H), (H, I))]
    lo, hi = nsplit.expert_range(E, world, rank)

    def owned(kind, l):
        return [torch.roll(pool[kind][(e + l) % 16], 1152 * (1 + e + 131 * l)) if lo <= e < hi else None for e in range(E)]

    layers = []
    for l in range(Lc):
        router = (torch.randn(H, E, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + l)) * 0.02)
        layers.append(be.MoeLayer(router, owned(0, l), owned(1, l), owned(2, l), k))
    if world > 1:
        layers[0].enable_expert_parallel(1, layers_per_epoch=Lc)
        for ly in layers[1:]:
            ly.enable_expert_parallel(1, share_with=layers[0])
    x0 = torch.randn(1, H, device=dev, generator=torch.Generator(device=dev).manual_seed(7))

    def one_token():
        x = x0
        for l, ly in enumerate(layers):
            y = ly.forward_ep(x, layer=l, bump_epoch=(l == 0)) if world > 1 else ly.forward(x)
            x = torch.nn.functional.layer_norm(y, (H,))  # one kernel: keeps magnitudes finite through 48 random layers
        return x

    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        out = one_token()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            out = one_token()
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
    be.device_status()
    ms = e0.elapsed_time(e1) / steps
    active = Lc * k * 3 * int(I * H * 144 / 256) + Lc * H * E * 4  # expert weights touched + routers, per token
    res = {"shape": "Qwen3-30B-A3B decode, 48 MoE layers (attention not run)", "ranks": world,
           "parallelism": "single GPU" if world == 1 else f"expert parallel x{world}",
           "ms_per_token": round(ms, 4), "us_per_layer": round(ms * 1e3 / Lc, 2), "layers_per_s": round(Lc * 1e3 / ms, 1),
           "weight_bytes_touched_per_token": active, "outputs_finite": bool(torch.isfinite(out).all().item()),
           "checksum": float(out.double().sum().item())}
    if world == 1:
        # cfg4's 256-token prefill through one layer: pairs sorted by expert, per-expert grouped GEMMs
        T = 256
        xp = torch.randn(T, H, device=dev)
        with torch.cuda.stream(stream):
            for ly in layers:  # every layer grows its scratch to 256 tokens here, outside the timed region
                ly.forward(xp)
            stream.synchronize()
            e0.record(stream)
            for ly in layers:
                yp = ly.forward(xp)
            e1.record(stream)
            stream.synchronize()
        be.device_status()
        pms = e0.elapsed_time(e1) / Lc
        res["prefill_256_tokens"] = {"ms_per_layer": round(pms, 4), "tokens_per_s_per_layer": round(T / pms * 1e3, 1),
                                     "pairs": T * k, "path": "pairs sorted by expert, per-expert grouped GEMM (exact)",
                                     "outputs_finite": bool(torch.isfinite(yp).all().item())}
    if world > 1:
        layers[0]._ep_buf.close()
    del layers, pool
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------
# prefill GEMM sweep (Q4_K weights, tensor-core path), reported beside the headline
# --------------------------------------------------------------------------
PREFILL_SWEEP = [(64, 24576, 4096), (256, 24576, 4096), (1024, 24576, 4096)]  # (M, N, K): fused gate+up projection
NOMINAL_INT8_TOPS = 4500.0  # dense int8, per GPU (nominal, for context)


def prefill_gemm_shapes(be, torch, dev, steps=10):
    """Q4_K x Q8_K GEMM through the device entry point (activation quantizer + tensor-core kernel per call), three
    distinct copies of the weight in rotation (170 MB > L2), CUDA events on the launching stream. Two kernels:
    "tensor_f16" (tcgen05 kind::f16 on operands dequantized to fp16; the default from 32 rows up) against the measured
    bf16 GEMM peaks of MEASURED_PEAKS.json, and "tensor" (tcgen05 kind::i8, integer sums exact) against the int8 rate
    measured now with a stream of the same MMA instruction; its tensor pipe does two passes (the 6-bit scale is split
    in two 8-bit operands), so mma = 2 x effective."""
    from oracle import oracle as O
    out = []
    rng = np.random.default_rng(11)
    peak_i8, clk_per_mma = be.measure_int8_peak()
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            mp = json.load(f)
        peak_f16, peak_f16_sus, src = float(mp["bf16_tflops"]), float(mp["bf16_tflops_sustained"]), "measured (cuBLAS bf16)"
    except Exception:
        peak_f16, peak_f16_sus, src = 1590.0, 1400.0, "fallback"
    for M, N, K in PREFILL_SWEEP:
        base = torch.from_numpy(O.random_q4_Kx8(rng, N, K)).to(dev)
        mats = [base, torch.roll(base, 4099 * 16), torch.roll(base, 2 * 4099 * 16)]
        A = torch.randn(M, K, device=dev)
        C = torch.empty(M, N, device=dev)
        ws = torch.empty(be.gemm_workspace_bytes("q4_K", M, N, K), dtype=torch.uint8, device=dev)
        row = {"M": M, "N": N, "K": K, "qtype": "q4_K"}
        for path in ("tensor_f16", "tensor"):
            be.set_gemm_path(path)
            for W in mats:
                be.gemm_q4_K(M, N, K, A, K, W, N, C, N, ws)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                for W in mats:
                    be.gemm_q4_K(M, N, K, A, K, W, N, C, N, ws)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (steps * len(mats))
            eff = 2.0 * M * N * K / (us * 1e-6) / 1e12
            if path == "tensor_f16":
                row["fp16_path"] = {"kernel": "tcgen05 kind::f16, fp16 operands", "us_per_call": round(us, 1),
                                    "TFLOP/s": round(eff, 1), "peak_TFLOP/s_burst": peak_f16,
                                    "peak_TFLOP/s_sustained": peak_f16_sus, "peak_source": src,
                                    "frac_of_burst_peak": round(eff / peak_f16, 4),
                                    "frac_of_sustained_peak": round(eff / peak_f16_sus, 4)}
            else:
                row["int8_path"] = {"kernel": "tcgen05 kind::i8, integer sums exact", "us_per_call": round(us, 1),
                                    "effective_TOP/s": round(eff, 1), "mma_TOP/s": round(2 * eff, 1),
                                    "int8_peak_TOP/s": round(peak_i8, 1),
                                    "int8_peak_source": "measured (tcgen05.mma kind::i8 stream)",
                                    "clk_per_128x256x32_mma": round(clk_per_mma, 1),
                                    "mma_frac_of_measured_int8": round(2 * eff / peak_i8, 4)}
        out.append(row)
        del mats, base, A, C, ws
        torch.cuda.empty_cache()
    # Q4_0 weights, same shapes: the fp16 kernel (its integer form would leave the tensor pipe every 32 of K);
    # Q6_K weights on the Qwen3-4B lm_head (N = 151936 ends inside a 256-row tile; 319 MB of weights, one copy)
    cases = [("q4_0", s) for s in PREFILL_SWEEP] + [("q6_K", (64, 151936, 2560)), ("q6_K", (256, 151936, 2560))]
    for qt, (M, N, K) in cases:
        if qt == "q4_0":
            base = torch.from_numpy(O.random_q4_0x8(rng, N, K)).to(dev)
            mats = [base, torch.roll(base, 4099 * 16), torch.roll(base, 2 * 4099 * 16)]
        else:
            base = torch.from_numpy(O.random_q6_K(rng, 4736, K)).to(dev).reshape(-1).repeat(N // 4736 + 1)
            base = base[:N * (K // 256) * 210].contiguous()
            mats = [base]
        gemm = be.gemm_q4_0 if qt == "q4_0" else be.gemm_q6_K
        A = torch.randn(M, K, device=dev)
        C = torch.empty(M, N, device=dev)
        ws = torch.empty(be.gemm_workspace_bytes(qt, M, N, K), dtype=torch.uint8, device=dev)
        be.set_gemm_path("tensor_f16")
        for W in mats:
            gemm(M, N, K, A, K, W, N, C, N, ws)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            for W in mats:
                gemm(M, N, K, A, K, W, N, C, N, ws)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (steps * len(mats))
        eff = 2.0 * M * N * K / (us * 1e-6) / 1e12
        out.append({"M": M, "N": N, "K": K, "qtype": qt,
                    "fp16_path": {"kernel": "tcgen05 kind::f16, fp16 operands", "us_per_call": round(us, 1),
                                  "TFLOP/s": round(eff, 1), "peak_TFLOP/s_burst": peak_f16,
                                  "peak_TFLOP/s_sustained": peak_f16_sus, "peak_source": src,
                                  "frac_of_burst_peak": round(eff / peak_f16, 4),
                                  "frac_of_sustained_peak": round(eff / peak_f16_sus, 4)}})
        del mats, base, A, C, ws
        torch.cuda.empty_cache()
    be.set_gemm_path("auto")
    be.device_status()
    return out


# --------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    from nntrainer_b200 import backend as be
    from nntrainer_b200 import build as nb_build

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        # a rank that dies must not leave the others in a collective for NCCL's default ten minutes
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=240))
    nb_build.build()
    be.init(local)
    dev = torch.device("cuda", local)

    base, how = make_base_weight()
    nsplit = world > 1 or args.nsplit

    def shard(r, i):
        """Weight shard of rank r for layer i: the base matrix with its row groups rotated (distinct memory per layer
        and per rank, same statistics)."""
        g = base.reshape(N_ROWS // 8, -1)
        return np.ascontiguousarray(np.roll(g, 11 * i + 5 * r, axis=0)).reshape(-1)

    host_ring = [shard(rank, i) for i in range(RING)]
    ring = [torch.from_numpy(w).to(dev) for w in host_ring]
    x0 = torch.from_numpy(np.random.default_rng(1).standard_normal(K_COLS).astype(np.float32)).to(dev)
    pdl = not args.no_pdl
    gathered = [torch.zeros(N_ROWS, device=dev) for _ in range(2)]
    group = None
    if nsplit:
        from nntrainer_b200.nsplit import NSplitGroup
        group = NSplitGroup(N_ROWS, RING, ring=args.gather_ring)

    def step_body():
        sp = int(torch.cuda.current_stream().cuda_stream)
        if group is not None:
            # N-split: every GEMV stores its slice into all ranks' gathered vectors; the next one takes as its activation
            # the slice its neighbour rank contributed, so every layer's input has crossed NVLink
            group.bump_epoch(sp)
            for i, W in enumerate(ring):
                xp = x0.data_ptr() if i == 0 else group.input_ptr(i, (rank + 1) % world)
                group.gemv("q4_K", K_COLS, xp, W.data_ptr(), i, sp, pdl=pdl, x_tagged=(i > 0))
            return
        src = x0  # every step restarts from the same input, then ping-pongs between two buffers
        for i, W in enumerate(ring):
            dst = gathered[i % 2]
            be.gemv("q4_K", N_ROWS, K_COLS, src, W, dst, pdl=pdl)
            src = dst

    def renorm():
        pass

    def verify_nsplit():
        """After a full pass: every rank holds the gathered outputs of the last two layers; recompute the last layer's
        slices of ALL ranks locally (plain single-GPU kernel) and require the same bits."""
        g_prev, g_last = group.gathered_numpy(RING - 2), group.gathered_numpy(RING - 1)
        for d in range(world):
            src = (d + 1) % world  # rank d read the slice its neighbour contributed
            xd = torch.from_numpy(g_prev[src * N_ROWS:(src + 1) * N_ROWS].copy()).to(dev)
            Wd = torch.from_numpy(shard(d, RING - 1)).to(dev)
            yd = torch.zeros(N_ROWS, device=dev)
            be.gemv("q4_K", N_ROWS, K_COLS, xd, Wd, yd)
            want = yd.cpu().numpy()
            got = g_last[d * N_ROWS:(d + 1) * N_ROWS]
            if not np.array_equal(want.view(np.uint32), got.view(np.uint32)):
                raise AssertionError(f"rank {rank}: gathered slice of rank {d} differs from the single-GPU kernel")
        be.device_status()
        return True

    # one CUDA graph per step (single GPU): the launch loop is otherwise bound by the host
    graph = None
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        step_body()
        stream.synchronize()
        verified = verify_nsplit() if group is not None else None
        if world > 1:
            dist.barrier()
        if not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step_body()

        def step():
            if graph is not None:
                graph.replay()
            else:
                step_body()

        for _ in range(max(args.warmup, 3)):
            step()
            renorm()
        stream.synchronize()
        clocks = Clocks(local)
        if rank == 0:
            clocks.start()
            time.sleep(0.3)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()  # after rank 0's sampler start-up, so that no rank's timed region contains it
            torch.cuda.synchronize()
        launches0 = be.launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        t1 = time.time()
        if world > 1:
            dist.barrier()
        ms = ev0.elapsed_time(ev1)
        launches = (be.launch_count() - launches0) if graph is None else RING * args.steps
        clk = clocks.stop(t0, t1) if rank == 0 else None
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        if group is not None:
            finite = bool(np.isfinite(group.gathered_numpy(RING - 1)).all())
            be.device_status()
            # the graph replays are where buffers are reused across passes: check the last pass as well
            verified = bool(verified) and verify_nsplit()
        else:
            finite = bool(torch.isfinite(gathered[0]).all() and torch.isfinite(gathered[1]).all())

    # ---- end to end through the host-pointer C ABI: host x in, host y out, per GEMV
    e2e = None
    if not args.no_e2e:  # every rank: its own slice of the global weight, host x in, host y slice out; max over ranks
        def all_ok(ok):  # every rank reaches this, whatever happened to it before
            if world == 1:
                return ok
            t = torch.tensor([0.0 if ok else 1.0], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item()) == 0.0

        err, registered = None, []
        try:
            # activation and result live where the plug-in's allocator puts the framework's tensors: page-locked memory
            xn = be.host_alloc((1, K_COLS), np.float32)
            yn = be.host_alloc((1, N_ROWS), np.float32)
            xn[...] = x0.cpu().numpy()[None]
            yn[...] = 0.0
            for W in host_ring:
                be.register_weight("q4_K", W, N_ROWS, K_COLS)
                registered.append(W)
            calls = [be.bind_gemm("q4_K", 1, N_ROWS, K_COLS, xn, K_COLS, W, N_ROWS, yn, N_ROWS) for W in host_ring]
            for _ in range(2):
                for call in calls:
                    call()
            torch.cuda.synchronize()
        except Exception as exc:  # noqa: BLE001
            err = f"{type(exc).__name__}: {exc}"[:300]
        e2e_steps = max(1, min(args.steps, 20))
        dt = 0.0
        if all_ok(err is None):
            if world > 1:
                dist.barrier()
            try:
                tt0 = time.perf_counter()
                for _ in range(e2e_steps):
                    for call in calls:
                        call()  # synchronous: the result is in yn when it returns
                        np.multiply(yn, 0.78, out=xn)  # chain on the host (one cheap pass; 0.78 keeps the magnitude level)
                torch.cuda.synchronize()
                dt = time.perf_counter() - tt0
            except Exception as exc:  # noqa: BLE001
                err = f"{type(exc).__name__}: {exc}"[:300]
            if world > 1:
                t = torch.tensor([dt], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dt = float(t.item())
        if all_ok(err is None) and dt > 0.0:
            e2e = {"value": round(world * e2e_steps * RING * ALG_BYTES / dt / 1e9, 2), "unit": "GB/s",
                   "h2d_bytes_per_step": world * RING * 4 * K_COLS, "d2h_bytes_per_step": world * RING * 4 * N_ROWS,
                   "us_per_call": round(dt / (e2e_steps * RING) * 1e6, 2),
                   "api": "nntr_cuda_gemm_q4_K (host pointers, weights cached in HBM)" +
                          ("" if world == 1 else "; every rank on its own row slice, host x in and host y slice out, no gather")}
        else:
            e2e = {"error": err or "the end-to-end leg failed on another rank"}
        for W in registered:
            be.unregister_weight(W)

    # the MoE decode step runs on every rank (expert parallel when there is more than one). A failure is recorded in the
    # line AND fails the run (exit code 3 after the line is printed)
    failures = []
    if e2e is not None and "error" in e2e:
        failures.append("e2e: " + e2e["error"])
    if group is not None and not verified:
        failures.append("n-split verification failed")
    moe = None
    if not args.no_moe:
        try:
            moe = moe_decode_step(be, torch, dev, world, rank)
        except Exception as exc:  # noqa: BLE001
            moe = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            failures.append("moe_decode_step: " + moe["error"])

    # every projection of the 4B shape sharded over the ranks (strong scaling), on every rank
    sharded = None
    if not args.no_extra and (world <= 2 or args.sharded_decode):
        try:
            sharded = decode_step_sharded(be, torch, dev, dist, world, rank, measured_peak()[0])
            if "error" not in sharded and not sharded["equals_single_gpu_chain"]:
                failures.append("decode_step_sharded: the gathered result differs from the single-GPU chain")
        except Exception as exc:  # noqa: BLE001  (recorded in the line; a side leg that could not run does not fail the run)
            sharded = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    if rank == 0:
        peak, which = measured_peak()
        total_bytes = world * args.steps * RING * ALG_BYTES
        value = total_bytes / (ms * 1e-3) / 1e9
        per_launch_us = ms * 1e3 / (args.steps * RING)
        achieved = ALG_BYTES / (per_launch_us * 1e-6) / 1e9
        others = other_shapes(be, torch, dev, peak) if (world == 1 and not args.no_extra) else None
        prefill = prefill_gemm_shapes(be, torch, dev) if (world == 1 and not args.no_extra) else None
        decode = decode_step_qwen3_4b(be, torch, dev, peak) if (world == 1 and not args.no_extra) else None
        model = model_decode_qwen3_4b(be, torch, dev, peak) if (world == 1 and not args.no_model) else None
        cpu_desc = None
        if world == 1 and not args.no_cpu:
            _, cpu_desc, _ = cpu_reference_gbps(host_ring, args.cpu_seconds)
        out = {"metric": "Q4_K GEMV HBM GB/s", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
               "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 5),
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
               "dtype": "u4xs8->s32, f32 scales", "data": "synthetic: " + how,
               "config": {"workload": WORKLOAD % RING,
                          "l2": "inputs larger than L2: %d MB of distinct weights per step" % (RING * WEIGHT_BYTES // 2**20),
                          "launch": ("CUDA graph, " if graph is not None else "eager, ") +
                                    ("programmatic dependent launch" if pdl else "plain launches"),
                          "parallelism": "single GPU" if group is None else
                          f"N-split x{world}: global weight [{world * N_ROWS}, {K_COLS}], output slices stored into every "
                          f"rank's gathered vector by the GEMV epilogue as (value, launch number) pairs over NVLink, no fence and no "
                          f"collective, verified={verified}",
                          "outputs_finite": finite,
                          # the side legs in short (the full records follow as extra keys of this line)
                          "moe_decode": None if not moe or "error" in moe else
                          {k: moe[k] for k in ("ranks", "ms_per_token", "us_per_layer", "checksum") if k in moe},
                          "moe_prefill_256": None if not moe or "error" in moe else moe.get("prefill_256_tokens"),
                          "dense_projections_tok_s": decode["tok/s"] if decode else None,
                          "dense_projections_sharded": None if not sharded else sharded if "error" in sharded else
                          {k: sharded[k] for k in ("ranks", "gathered_buffers", "ms_per_token", "plain_chain_ms_per_token", "tok/s",
                                                   "frac_of_aggregate_hbm_peak", "equals_single_gpu_chain")},
                          "model_decode_tok_s": model["tok/s"] if model else None,
                          "model_decode_tokens_equal_cpu": model["first_tokens_equal_cpu"] if model else None,
                          "failures": failures},
               "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                            "frac": round(achieved / peak, 4), "peak_source": which + " (copy bandwidth)",
                            "us_per_launch": round(per_launch_us, 4),
                            "traffic": args.traffic if args.traffic is not None else NCU_TRAFFIC_BYTES,
                            "kernel": "gemv_q4_K_resident_kernel", "algorithmic_bytes_per_launch": ALG_BYTES},
               "cpu_baseline": cpu_desc, "e2e": e2e, "gpu_launches": int(launches), "clocks": clk,
               "other_decode_gemv_shapes": others, "prefill_gemm_sweep": prefill,
               "decode_step": decode, "decode_step_sharded": sharded, "model_decode": model, "moe_decode_step": moe}
        print(json.dumps(out), flush=True)
    if group is not None:
        group.close()
    if world > 1:
        dist.destroy_process_group()
    if failures:
        sys.stderr.write("bench: " + "; ".join(failures) + "\n")
        sys.exit(3)


def run_case(args):
    """Small single-kernel cases for profiler captures (a few hundred MB on the device, a handful of launches)."""
    import torch
    from nntrainer_b200 import backend as be
    from nntrainer_b200 import build as nb_build
    from oracle import oracle as O
    nb_build.build()
    be.init(0)
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(3)
    reps = max(1, args.steps if args.steps < 100 else 5)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.case in ("prefill", "prefill_f16"):
        M, N, K = (512, 4096, 4096) if args.case == "prefill" else (256, 24576, 4096)
        W = torch.from_numpy(O.random_q4_Kx8(rng, N, K)).to(dev)
        A = torch.randn(M, K, device=dev)
        C = torch.empty(M, N, device=dev)
        ws = torch.empty(be.gemm_workspace_bytes("q4_K", M, N, K), dtype=torch.uint8, device=dev)
        be.set_gemm_path("tensor" if args.case == "prefill" else "tensor_f16")
        call = lambda: be.gemm_q4_K(M, N, K, A, K, W, N, C, N, ws)
        work = {"case": args.case, "M": M, "N": N, "K": K, "qtype": "q4_K", "ops": 2.0 * M * N * K}
    elif args.case == "lm_head_prefill":
        M, N, K = 256, 151936, 2560
        W = torch.from_numpy(O.random_q6_K(rng, N, K)).to(dev)
        A = torch.randn(M, K, device=dev)
        C = torch.empty(M, N, device=dev)
        ws = torch.empty(be.gemm_workspace_bytes("q6_K", M, N, K), dtype=torch.uint8, device=dev)
        be.set_gemm_path("tensor_f16")
        call = lambda: be.gemm_q6_K(M, N, K, A, K, W, N, C, N, ws)
        work = {"case": args.case, "M": M, "N": N, "K": K, "qtype": "q6_K", "ops": 2.0 * M * N * K}
    elif args.case == "moe_layer":
        H, I, E, k = 2048, 768, 128, 8
        mk = lambda n, kk: torch.from_numpy(O.random_q4_Kx8(rng, n, kk)).to(dev)
        pool = [(mk(I, H), mk(I, H), mk(H, I)) for _ in range(8)]
        layer = be.MoeLayer(torch.randn(H, E, device=dev) * 0.02, [pool[e % 8][0] for e in range(E)],
                            [pool[e % 8][1] for e in range(E)], [pool[e % 8][2] for e in range(E)], k)
        x = torch.randn(1, H, device=dev)
        call = lambda: layer.forward(x)
        work = {"case": "moe_layer", "hidden": H, "inter": I, "experts": E, "top_k": k, "tokens": 1}
    elif args.case == "decoder":
        # four layers of the Qwen3-4B shape with the full vocabulary, 512 cache rows in place of a prefill; steps run
        # eagerly so that a profiler sees every launch of a token
        import os
        import tempfile
        from nntrainer_b200.decoder import DecoderConfig, Qwen3Decoder
        from oracle.cpu_decoder import synthetic_weights, write_bin
        context = 512
        cfg = DecoderConfig(n_layers=4, hidden=2560, n_heads=32, n_kv_heads=8, head_dim=128, inter=9728, vocab=151936,
                            max_seq=context + 64)
        w = synthetic_weights(cfg, seed=5)
        with tempfile.TemporaryDirectory() as td:
            path = os.path.join(td, "decoder_case.bin")
            write_bin(path, cfg, w)
            dec = Qwen3Decoder(cfg, path, pdl=True)
        for a in dec.attn:
            a.kcache[:context].copy_((torch.randn((context, cfg.n_kv_heads, cfg.head_dim), device=dev) * 0.5).half())
            a.vcache[:context].copy_((torch.randn((context, cfg.n_kv_heads, cfg.head_dim), device=dev) * 0.5).half())
        tok = torch.full((1,), 11.0, device=dev)
        state = {"pos": context}

        def call():
            nxt, nxt_f = dec.step(tok, state["pos"])
            tok.copy_(nxt_f)
            state["pos"] += 1
        work = {"case": "decoder", "layers": cfg.n_layers, "hidden": cfg.hidden, "vocab": cfg.vocab, "context": context,
                "launches_per_token": 1 + cfg.n_layers * 7 + 3}
    else:  # lm_head
        N, K = 151936, 2560
        W = torch.from_numpy(O.random_q6_K(rng, N, K)).to(dev)
        x = torch.randn(1, K, device=dev)
        y = torch.empty(1, N, device=dev)
        call = lambda: be.gemm_q6_K(1, N, K, x, K, W, N, y, N)
        work = {"case": "lm_head", "N": N, "K": K, "qtype": "q6_K", "bytes": N * (K // 256) * 210 + 4 * K + 4 * N}
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        call()
    e1.record()
    torch.cuda.synchronize()
    be.device_status()
    work["us_per_call"] = round(e0.elapsed_time(e1) * 1e3 / reps, 2)
    print(json.dumps(work))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch")
    ap.add_argument("--nsplit", action="store_true", help="run the N-split exchange path even on one GPU")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the other decode GEMV shapes")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-pointer end-to-end leg (profiling runs)")
    ap.add_argument("--no-moe", action="store_true", help="skip the MoE decode step")
    ap.add_argument("--no-model", action="store_true", help="skip the whole-model decode leg")
    ap.add_argument("--sharded-decode", action="store_true",
                    help="run the row-sharded projection chain of the 4B shape on more than two GPUs too (default: one "
                         "and two)")
    ap.add_argument("--gather-ring", type=int, default=4, help="gathered buffers in rotation on the N-split path (2: exchange in "
                    "the streaming kernel; 4: in the resident-weights kernel)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--ring", type=int, default=RING, help="distinct weight matrices per step (default keeps every launch out of L2)")
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch of the GEMV kernel from an ncu capture (reported as roofline.traffic)")
    ap.add_argument("--case", default=None, choices=["prefill", "prefill_f16", "lm_head", "lm_head_prefill", "moe_layer", "decoder"],
                    help="run one small single-kernel case (profiler captures) instead of the benchmark")
    args = ap.parse_args()
    globals()["RING"] = args.ring
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
