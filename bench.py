#!/usr/bin/env python3
"""Decode and prefill throughput of gguf2bin_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode|ragged8|b64|senotar|levolix|sominex|mopitar] [--batch B] [--layers L] [--context C]
                    [--no-points] [--sizes 0.6b|8b|14b]

The default run has the layer sizes of Qwen3-0.6B (28 layers, width 1024, 16/8 heads of
128, feed-forward 3072, vocabulary 151936, tied embeddings) with random bfloat16
weights, a batch of 8 and a context of 4096: every sequence is prefilled with random
token ids up to position 2048 and then decoded.  A "step" is one decode step of the
whole batch.  It prints ONE JSON line:

  value      decoded tokens per second over exactly K steps, timed on the device with CUDA
             events (the steps run back to back from a CUDA graph; sampled tokens stay on
             the device)
  e2e        the same through the Python entry point (LLM.generate; `default_sampling`: with its own
             sampling parameters instead of greedy): token ids go in
             from pinned host memory and come back to the host every step; the median of
             three calls (each with its own prompts' prefill before and the set-up of its
             decode session inside the timed steps), all three listed under "runs"
  prefill    one step over a 2,048-token prompt: tokens per second, milliseconds (the median of
             three runs that replay the shape's graph; ``plain_ms`` is a run of the warm engine
             without the graph, what a shape costs when it is first seen; ``first_ms`` the very
             first run, which also builds scratch buffers and loads kernels), and the fraction of
             the tensor-core peak its flops reach
  roofline   bytes a decode step must read (every weight once, the cache of the live
             requests) divided by its time, against the measured copy bandwidth
  points     decode tokens per second at batch 1 and 64 (fewer steps), each with its step time
             and its own roofline figures

``--workload ragged8`` runs the workload of the Qwen3-8B configuration (all 36 layers): eight
prompts with lengths drawn uniformly from [128, 2048] (seeded) in ONE ragged prompt step, whose
tokens per second go under ``prefill``, then 256 decode steps.  ``--workload b64`` runs that of
the Qwen3-14B configuration (all 40 layers): 64 prompts of 512 tokens in one prompt step, then
decoding to a context of 2,048.  The weights are made in device memory (no folder is written).

``--workload senotar`` is a comparison, not the benchmark: at three layer sizes it builds a
Senotar model (latent attention, gated residuals, xIELU feed-forward) and a Qwen3 model with the
same width, layer count, vocabulary and (within 3 %) parameter count, and times for each one
prompt step of 2,048 tokens and decode steps at batch 8 behind 2,048-token prompts, on the
device, with the fraction of the tensor-core peak (prompt) and of the copy bandwidth (decode)
that each reaches.  It prints one JSON line of its own shape.

``--workload levolix`` is the same kind of comparison for Levolix (retention layers and layers with
chunked attention beside the gated delta rule, routed experts): active parameters per token within
a few per cent of the Qwen3 model's; the decode roofline counts every expert matrix once, the
states read and written, and the keys and values of a request's current chunk.

``--workload mopitar`` sets Mopitar (two score maps per head behind a window with kept first tokens, capped
attention with a sink beside a selective state-space branch, layers that borrow keys and values, routed
experts in groups) beside Sominex, the library's closest design (one norm in front of both sublayers,
windowed attention, a state-space mixer, routed experts with a shared one), at equal width, layer count,
vocabulary and, within a few per cent, active parameters.

Peaks come from MEASURED_PEAKS.json beside this file when present, else from the
fallback figures 6.65 TB/s and 1.59 PFLOP/s.  Inputs are synthetic.  Between timed steps
nothing is flushed: a step reads more than a gigabyte of weights and cache, far more than
the 126 MB of L2.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_0P6B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=1024, intermediate_size=3072,
                  num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                  head_dim=128, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                  tie_word_embeddings=True, max_position_embeddings=40960)
# the layer sizes of Qwen3-8B and Qwen3-14B, for `--sizes` (not the default run)
OTHER_SIZES = {
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, tie_word_embeddings=False),
    "14b": dict(hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40,
                num_key_value_heads=8, head_dim=128, tie_word_embeddings=False),
}
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                        source="measured")
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None,
                    sm_max_mhz=max(mx) if mx else None, reasons=sorted(reasons),
                    samples=len(sm))


def model_bytes_and_flops(cfg: dict, n_layers: int):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    nq, nk = nh * hd, nkv * hd
    layer = H * (nq + 2 * nk) + nq * H + 2 * H * I + I * H            # matrix parameters of a layer
    vectors = 2 * H + 2 * hd
    weight_bytes = 2 * (n_layers * (layer + vectors) + H + V * H)       # bf16; lm_head read once
    kv_bytes_per_token = 2 * nk * 2 * n_layers                          # K and V, bf16, all layers
    return dict(layer_params=layer, weight_bytes=weight_bytes, kv_bytes_per_token=kv_bytes_per_token,
                nq=nq)


def prefill_flops(cfg: dict, n_layers: int, lengths) -> float:
    """Flops of one prompt step over sequences of these lengths, logits at each one's last place."""
    m = model_bytes_and_flops(cfg, n_layers)
    total = float(sum(lengths))
    linear = 2.0 * total * n_layers * m["layer_params"]
    attention = sum(n_layers * 4.0 * m["nq"] * T * (T + 1) / 2 for T in lengths)
    head = 2.0 * cfg["vocab_size"] * cfg["hidden_size"] * len(lengths)
    return linear + attention + head


def random_prompts(n: int, length: int, vocab: int, seed: int):
    import numpy as np
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, length).tolist() for _ in range(n)]


def timed_prompt_step(llm, prompts, repeats: int):
    """Milliseconds of ONE step over all the prompts (logits at each last place), device-timed:
    (the very first run, which also builds scratch buffers and loads kernels; the median of the
    last ``repeats`` runs, which replay the shape's graph; a run of the warm engine without the
    graph, which is what a shape costs the first time it is seen)."""
    import gc
    import torch
    from gguf2bin_b200.engine import StepEntry
    times = []
    # the plain run's time is the host's; a collection of Python's cycle collector in the middle of it
    # (this program holds hundreds of thousands of token ids in lists) adds a millisecond or two
    gc.collect()
    gc.disable()
    for i in range(3 + repeats + 1):
        if i == 3 + repeats:                       # once more without the graph: a warm engine's plain run,
            graphs, llm.engine.step_graphs = llm.engine.step_graphs, False     # what a shape seen for the first time costs
        seqs = [llm.open_sequence() for _ in prompts]
        for s, p in zip(seqs, prompts):
            llm.engine.cache.reserve(s, len(p))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        llm.step([StepEntry(s, p, (len(p) - 1,)) for s, p in zip(seqs, prompts)])
        e1.record()
        torch.cuda.synchronize()
        for s in seqs:
            llm.close_sequence(s)
        times.append(e0.elapsed_time(e1))
    llm.engine.step_graphs = graphs
    gc.enable()
    return times[0], statistics.median(times[3:-1]), times[-1]


def decode_device_timed(llm, prompts, steps: int, warmup: int, vocab: int, whole_batch_prefill: bool):
    """Decodes ``steps`` steps after the prompts and ``warmup`` untimed steps: (seconds for
    exactly ``steps`` steps, launches per step, mean context over the timed steps), timed on
    the device.  The prompts are prefilled one sequence per step, or all in one ragged step."""
    import torch
    from gguf2bin_b200.engine import DecodeSession, StepEntry
    from gguf2bin_b200.sampling import Sampler, SamplingParams
    eng = llm.engine
    batch = len(prompts)
    seqs = [eng.open_sequence() for _ in range(batch)]
    try:
        for s, p in zip(seqs, prompts):
            eng.cache.reserve(s, len(p) + warmup + steps + 1)
        if whole_batch_prefill:
            eng.step([StepEntry(s, p, ()) for s, p in zip(seqs, prompts)])
        else:
            for s, p in zip(seqs, prompts):
                eng.step([StepEntry(s, p, ())])
        sampler = Sampler(eng.cache.seq_state, eng.device)
        session = DecodeSession(eng, seqs, sampler, SamplingParams.plain(0.0), use_graph=True,
                                eager_steps=1)
        session.set_tokens(random_prompts(1, batch, vocab, 7)[0])
        for _ in range(warmup):
            session.run()
        torch.cuda.synchronize()
        start = sum(s.length for s in seqs) / batch
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            session.run()
        t1.record()
        torch.cuda.synchronize()
        eng.check()
        return t0.elapsed_time(t1) / 1e3, session.launches_per_step, start + steps / 2.0
    finally:
        for s in seqs:
            eng.close_sequence(s)


def hbm_roofline(sizes: dict, batch: int, mean_ctx: float, sec_per_step: float, pk: dict) -> dict:
    """Bytes a decode step has to read (every weight once, the cache of the live requests)
    over its time, against the copy bandwidth."""
    step_bytes = sizes["weight_bytes"] + batch * mean_ctx * sizes["kv_bytes_per_token"]
    achieved = step_bytes / sec_per_step / 1e9
    return dict(bound="hbm", achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s",
                frac=achieved / pk["hbm_gbs"], peaks=pk["source"])


# ---- Senotar beside Qwen3 at equal sizes --------------------------------------------------------
# name: (width, heads, qk/v size per head, latent rank, Senotar's ff; Qwen3's kv heads, head size, ff)
EQUAL_SIZES = {
    "w1024": (1024, 16, 64, 128, 5632, 8, 128, 3072),
    "w2048": (2048, 16, 128, 128, 8192, 8, 128, 6144),
    "w4096": (4096, 32, 128, 128, 15360, 8, 128, 12288),
}


def senotar_config(width, heads, dim, rank, ff, layers, vocab) -> dict:
    """Every second layer attends over the latents of the layer in front of it."""
    out = []
    for i in range(layers):
        mixer = dict(heads=heads, dim=dim, vdim=dim, kv_rank=rank, scale=dim ** -0.5)
        if i % 2:
            mixer["kv_from"] = i - 1
        out.append(dict(type="latent_attention", mixer=mixer, mlp=dict(kind="dense", ff=ff)))
    return dict(architecture="Senotar", width=width, vocab=vocab, norm=dict(eps=1e-6), canon=dict(taps=3),
                embedding=dict(scale=float(width) ** 0.5, bigram=dict(buckets=100003, mul_prev=131, mul_cur=5)),
                layers=out)


def senotar_bytes_and_flops(cfg: dict) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    params, cache_bytes_per_token, attn = 0, 0, 0
    for layer in cfg["layers"]:
        m, ff = layer["mixer"], layer["mlp"]["ff"]
        H, dk, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
        params += W * (H * dk + H) + H * dk * r + H * dv * r + W * H * dv + 2 * W * W + 2 * W * ff
        if "kv_from" not in m:
            params += r * W
        cache_bytes_per_token += 2 * r              # every layer's attention reads the latents it attends over
        attn += 4 * H * r                           # flops per (query, key) pair: scores and sums, both of rank r
    return dict(layer_params=params, weight_bytes=2 * (params + V * W), kv_bytes_per_token=cache_bytes_per_token,
                attn_flops_per_pair=attn)


def senotar_comparison(a, pk) -> int:
    import torch
    from gguf2bin_b200.api import LLM
    layers, vocab, batch, T = a.layers or 8, 151936, a.batch or 8, a.prefill_tokens
    steps, warmup = a.steps or 128, max(a.warmup, 8)
    max_tokens = batch * (T + warmup + steps + 128)
    rows = {}
    clocks = ClockSampler()
    clocks.start()
    for name, (width, heads, dim, rank, ff, q_kv, q_hd, q_ff) in EQUAL_SIZES.items():
        if a.sizes_only and name not in a.sizes_only.split(","):
            continue
        row = {}
        for arch in ("senotar", "qwen3"):
            if arch == "senotar":
                cfg = senotar_config(width, heads, dim, rank, ff, layers, vocab)
                sizes = senotar_bytes_and_flops(cfg)
                flops = 2.0 * T * sizes["layer_params"] + sizes["attn_flops_per_pair"] * T * (T + 1) / 2 + 2.0 * vocab * width
            else:
                cfg = dict(QWEN3_0P6B, hidden_size=width, intermediate_size=q_ff, num_hidden_layers=layers,
                           num_attention_heads=heads, num_key_value_heads=q_kv, head_dim=q_hd, vocab_size=vocab,
                           tie_word_embeddings=False)
                sizes = model_bytes_and_flops(cfg, layers)
                sizes["layer_params"] *= layers
                flops = prefill_flops(cfg, layers, [T])
            llm = LLM.random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_seqs=batch + 1)
            first, ms, plain = timed_prompt_step(llm, random_prompts(1, T, vocab, 1), repeats=3)
            sec, per_step, mean_ctx = decode_device_timed(llm, random_prompts(batch, T, vocab, 100), steps, warmup,
                                                          vocab, whole_batch_prefill=False)
            roof = hbm_roofline(sizes, batch, mean_ctx, sec / steps, pk)
            row[arch] = dict(
                parameters_per_layer_m=round(sizes["layer_params"] / layers / 1e6, 1),
                prefill_tokens_per_s=round(T / (ms / 1e3)), prefill_ms=round(ms, 3), prefill_plain_ms=round(plain, 3),
                prefill_frac_of_tensor_peak=round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
                decode_tokens_per_s=round(batch * steps / sec), decode_ms_per_step=round(sec / steps * 1e3, 4),
                decode_launches_per_step=per_step, decode_gbs=round(roof["achieved"]),
                decode_frac_of_copy_bandwidth=round(roof["frac"], 3))
            del llm
            torch.cuda.empty_cache()
        rows[name] = row
    print(json.dumps({"metric": "prefill and decode tokens/s of Senotar beside Qwen3 at equal sizes (random weights)",
                      "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "impl": "ours",
                      "config": {"layers": layers, "vocab": vocab, "prompt_tokens": T, "decode_batch": batch,
                                 "decode_context_from": T + warmup, "decode_steps": steps, "peaks": pk["source"],
                                 "l2": "inputs larger than L2 (weights + cache read every step)"},
                      "sizes": rows, "clocks": clocks.stop()}))
    return 0


# ---- Levolix beside Qwen3 at equal sizes ----------------------------------------------------------
# name: (width, retention heads / key size / value size, attention heads / kv heads / head size / chunk,
#        delta-rule heads / query-key heads / key size / value size, experts / identity / top / expert ff;
#        Qwen3's heads, kv heads, head size, ff)
LEVOLIX_SIZES = {
    "w1024": (1024, (4, 128, 256), (8, 4, 128, 512), (4, 2, 128, 128), (16, 2, 4, 768), 16, 8, 128, 3072),
    "w2048": (2048, (8, 128, 256), (16, 8, 128, 512), (8, 4, 128, 128), (16, 2, 4, 1536), 16, 8, 128, 6144),
    "w4096": (4096, (16, 128, 256), (32, 8, 128, 512), (16, 4, 128, 128), (16, 2, 4, 3072), 32, 8, 128, 12288),
}


def levolix_config(width, ret, att, delta, moe, layers, vocab) -> dict:
    """Two retention layers, then one with attention and the delta rule side by side, and so on."""
    out = []
    mlp = dict(kind="moe", expert=dict(ff=moe[3]), router=dict(experts=moe[0], identity=moe[1], top=moe[2]))
    for i in range(layers):
        if i % 3 < 2:
            H, D, V = ret
            decay = [1.0 - 2.0 ** (-5 - 6.0 * h / max(1, H - 1)) for h in range(H)]
            out.append(dict(type="retention", mlp=mlp,
                            mixer=dict(heads=H, dim=D, vdim=V, decay=decay, rot=dict(dims=D, base=1e6))))
        else:
            H, G, D, chunk = att
            left = dict(heads=H, kv_heads=G, dim=D, vdim=D, mask=dict(size=chunk), rot=dict(dims=D, base=5e4), scale=D ** -0.5)
            right = dict(heads=delta[0], kv_heads=delta[1], dim=delta[2], vdim=delta[3], conv=4)
            out.append(dict(type="parallel", mlp=mlp, mixer=dict(left=left, right=right, left_scale=1.0, right_scale=1.0)))
    return dict(architecture="Levolix", width=width, vocab=vocab, norm=dict(eps=1e-6), layers=out)


def levolix_bytes_and_flops(cfg: dict) -> dict:
    """Parameters a token's step multiplies by (the chosen experts only), the bytes a decode step of a
    batch reads at least (every matrix once: a batch of 8 with 4 choices each touches most experts),
    and what every live request adds (keys and values of its chunk, its states)."""
    W, V = cfg["width"], cfg["vocab"]
    active = total = state_bytes = kv_per_token = attn = 0
    for layer in cfg["layers"]:
        m, mlp = layer["mixer"], layer["mlp"]
        if layer["type"] == "retention":
            mix = W * m["heads"] * (2 * m["dim"] + 3 * m["vdim"])
            state_bytes += 2 * 4 * m["heads"] * m["dim"] * m["vdim"]                 # read and written
        else:
            l, r = m["left"], m["right"]
            mix = W * (2 * l["heads"] * l["dim"] + 2 * l["kv_heads"] * l["dim"] + 2 * l["heads"] * l["vdim"])
            mix += W * (2 * r["kv_heads"] * r["dim"] + 3 * r["heads"] * r["vdim"] + 2 * r["heads"])
            state_bytes += 2 * 4 * r["heads"] * r["dim"] * r["vdim"]
            kv_per_token += 2 * 2 * l["kv_heads"] * l["dim"]
            attn += 4 * l["heads"] * l["dim"]
        e = mlp["router"]
        one = 3 * W * mlp["expert"]["ff"]
        real_share = e["experts"] / (e["experts"] + e["identity"])
        active += mix + W * (e["experts"] + e["identity"]) + one * e["top"] * real_share
        total += mix + W * (e["experts"] + e["identity"]) + one * e["experts"]
    return dict(layer_params=active, total_params=total, weight_bytes=2 * (total + V * W), state_bytes=state_bytes,
                kv_bytes_per_token=kv_per_token, attn_flops_per_pair=attn)


def levolix_comparison(a, pk) -> int:
    import torch
    from gguf2bin_b200.api import LLM
    layers, vocab, batch, T = a.layers or 6, 151936, a.batch or 8, a.prefill_tokens
    steps, warmup = a.steps or 128, max(a.warmup, 8)
    max_tokens = batch * (T + warmup + steps + 128)
    rows = {}
    clocks = ClockSampler()
    clocks.start()
    for name, (width, ret, att, delta, moe, q_heads, q_kv, q_hd, q_ff) in LEVOLIX_SIZES.items():
        if a.sizes_only and name not in a.sizes_only.split(","):
            continue
        row = {}
        for arch in ("levolix", "qwen3"):
            if arch == "levolix":
                cfg = levolix_config(width, ret, att, delta, moe, layers, vocab)
                sizes = levolix_bytes_and_flops(cfg)
                chunk = att[3]
                pairs = sum(min(t % chunk, t) + 1 for t in range(T))        # keys a token sees: its chunk only
                flops = 2.0 * T * sizes["layer_params"] + sizes["attn_flops_per_pair"] * pairs + 2.0 * vocab * width
                extra = batch * sizes["state_bytes"]
                ctx_cap = chunk / 2.0
            else:
                cfg = dict(QWEN3_0P6B, hidden_size=width, intermediate_size=q_ff, num_hidden_layers=layers,
                           num_attention_heads=q_heads, num_key_value_heads=q_kv, head_dim=q_hd, vocab_size=vocab,
                           tie_word_embeddings=True)
                sizes = model_bytes_and_flops(cfg, layers)
                sizes["weight_bytes"] -= 2 * vocab * width               # tied: the table is the head
                sizes["layer_params"] *= layers
                flops = prefill_flops(cfg, layers, [T])
                extra, ctx_cap = 0, None
            llm = LLM.random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_seqs=batch + 1)
            first, ms, plain = timed_prompt_step(llm, random_prompts(1, T, vocab, 1), repeats=3)
            sec, per_step, mean_ctx = decode_device_timed(llm, random_prompts(batch, T, vocab, 100), steps, warmup,
                                                          vocab, whole_batch_prefill=False)
            step_bytes = sizes["weight_bytes"] + extra + batch * (min(mean_ctx, ctx_cap) if ctx_cap else mean_ctx) \
                * sizes["kv_bytes_per_token"]
            gbs = step_bytes / (sec / steps) / 1e9
            row[arch] = dict(
                active_parameters_per_layer_m=round(sizes["layer_params"] / layers / 1e6, 1),
                prefill_tokens_per_s=round(T / (ms / 1e3)), prefill_ms=round(ms, 3), prefill_plain_ms=round(plain, 3),
                prefill_frac_of_tensor_peak=round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
                decode_tokens_per_s=round(batch * steps / sec), decode_ms_per_step=round(sec / steps * 1e3, 4),
                decode_launches_per_step=per_step, decode_step_mb=round(step_bytes / 1e6, 1), decode_gbs=round(gbs),
                decode_frac_of_copy_bandwidth=round(gbs / pk["hbm_gbs"], 3))
            del llm
            torch.cuda.empty_cache()
        rows[name] = row
    print(json.dumps({"metric": "prefill and decode tokens/s of Levolix beside Qwen3 at equal sizes (random weights)",
                      "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "impl": "ours",
                      "config": {"layers": layers, "vocab": vocab, "prompt_tokens": T, "decode_batch": batch,
                                 "decode_context_from": T + warmup, "decode_steps": steps, "peaks": pk["source"],
                                 "l2": "inputs larger than L2 (weights, states and cache read every step)"},
                      "sizes": rows, "clocks": clocks.stop()}))
    return 0


# ---- Sominex beside Qwen3 at equal sizes ----------------------------------------------------------
# name: (width, attention heads / kv heads / head size / window / block, state-space heads / groups / state / value size,
#        mLSTM heads / key size / value size, dense ff, experts / top / expert ff / shared ff;
#        Qwen3's heads, kv heads, head size, ff)
SOMINEX_SIZES = {
    "w1024": (1024, (8, 4, 128, 512, 64), (32, 4, 128, 64), (4, 128, 256), 3072, (16, 2, 768, 1536), 16, 8, 128, 3072),
    "w2048": (2048, (16, 8, 128, 512, 64), (64, 8, 128, 64), (8, 128, 256), 6144, (16, 2, 1536, 3072), 16, 8, 128, 6144),
    "w4096": (4096, (32, 8, 128, 512, 64), (128, 8, 128, 64), (16, 128, 256), 12288, (16, 2, 3072, 6144), 32, 8, 128, 12288),
}


def sominex_config(width, att, ssm, mls, ff, moe, layers, vocab) -> dict:
    """Attention, state space, mLSTM in turn; dense and routed feed-forwards in turn."""
    out = []
    dense = dict(kind="dense", ff=ff, limit=7.0)
    routed = dict(kind="moe", expert=dict(ff=moe[2]), router=dict(experts=moe[0], top=moe[1], scale=2.5), shared=dict(ff=moe[3]))
    for i in range(layers):
        mlp = routed if i % 2 else dense
        if i % 3 == 0:
            H, G, D, window, pool = att
            scaling = dict(factor=4.0, original=2048, fast=32.0, slow=1.0)
            out.append(dict(type="attention", mlp=mlp,
                            mixer=dict(heads=H, kv_heads=G, dim=D, vdim=D, scale=D ** -0.5, mask=dict(size=window, pool=pool),
                                       rot=dict(dims=D // 2, base=1e6, scaling=scaling))))
        elif i % 3 == 1:
            H, G, N, V = ssm
            out.append(dict(type="mamba2", mlp=mlp, mixer=dict(heads=H, groups=G, state=N, vdim=V, conv=4, norm_groups=G)))
        else:
            H, D, V = mls
            out.append(dict(type="mlstm", mlp=mlp, mixer=dict(heads=H, dim=D, vdim=V, gate_cap=15.0)))
    return dict(architecture="Sominex", width=width, vocab=vocab, norm=dict(eps=1e-5), embedding=dict(scale=1.0), layers=out)


def sominex_bytes_and_flops(cfg: dict, T: int) -> dict:
    """Parameters a token's step multiplies by (the chosen experts and the shared one), the bytes a decode
    step of a batch reads at least (every matrix once, every state read and written, the window's keys
    and the blocks' means in front of it), and the (query, key) pairs of a prompt of T tokens."""
    W, V = cfg["width"], cfg["vocab"]
    active = total = state_bytes = 0
    attn_layers = []
    pair_flops = 0.0
    for layer in cfg["layers"]:
        m, mlp = layer["mixer"], layer["mlp"]
        if layer["type"] == "attention":
            mix = W * (2 * m["heads"] * m["dim"] + 2 * m["kv_heads"] * m["dim"])
            attn_layers.append((2 * 2 * m["kv_heads"] * m["dim"], m["mask"]["size"], m["mask"]["pool"]))
            pairs = sum(min(t + 1, m["mask"]["size"]) + max(0, (t - m["mask"]["size"] + 1) // m["mask"]["pool"]) for t in range(T))
            pair_flops += 4.0 * m["heads"] * m["dim"] * pairs
        elif layer["type"] == "mamba2":
            inner = m["heads"] * m["vdim"]
            mix = W * (3 * inner + 2 * m["groups"] * m["state"] + m["heads"])
            state_bytes += 2 * 4 * m["heads"] * m["state"] * m["vdim"]
        else:
            mix = W * m["heads"] * (2 * m["dim"] + 3 * m["vdim"] + 2)
            state_bytes += 2 * 4 * m["heads"] * m["dim"] * (m["vdim"] + 1)
        if mlp["kind"] == "dense":
            a = t = 3 * W * mlp["ff"]
        else:
            r = mlp["router"]
            a = W * r["experts"] + 3 * W * (mlp["expert"]["ff"] * r["top"] + mlp["shared"]["ff"])
            t = W * r["experts"] + 3 * W * (mlp["expert"]["ff"] * r["experts"] + mlp["shared"]["ff"])
        active += mix + a
        total += mix + t

    def kv_bytes(ctx: float) -> float:
        return sum(b * (min(ctx, w) + max(0.0, ctx - w) / p) for b, w, p in attn_layers)
    return dict(layer_params=active, total_params=total, weight_bytes=2 * (total + 2 * V * W), state_bytes=state_bytes,
                kv_bytes=kv_bytes, pair_flops=pair_flops)


def sominex_comparison(a, pk) -> int:
    import torch
    from gguf2bin_b200.api import LLM
    layers, vocab, batch, T = a.layers or 6, 151936, a.batch or 8, a.prefill_tokens
    steps, warmup = a.steps or 128, max(a.warmup, 8)
    max_tokens = batch * (T + warmup + steps + 128)
    rows = {}
    clocks = ClockSampler()
    clocks.start()
    for name, (width, att, ssm, mls, ff, moe, q_heads, q_kv, q_hd, q_ff) in SOMINEX_SIZES.items():
        if a.sizes_only and name not in a.sizes_only.split(","):
            continue
        row = {}
        for arch in ("sominex", "qwen3"):
            if arch == "sominex":
                cfg = sominex_config(width, att, ssm, mls, ff, moe, layers, vocab)
                sizes = sominex_bytes_and_flops(cfg, T)
                flops = 2.0 * T * sizes["layer_params"] + sizes["pair_flops"] + 2.0 * vocab * width
            else:
                cfg = dict(QWEN3_0P6B, hidden_size=width, intermediate_size=q_ff, num_hidden_layers=layers,
                           num_attention_heads=q_heads, num_key_value_heads=q_kv, head_dim=q_hd, vocab_size=vocab,
                           tie_word_embeddings=False)
                sizes = model_bytes_and_flops(cfg, layers)
                sizes["layer_params"] *= layers
                flops = prefill_flops(cfg, layers, [T])
            llm = LLM.random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_seqs=batch + 1)
            first, ms, plain = timed_prompt_step(llm, random_prompts(1, T, vocab, 1), repeats=3)
            sec, per_step, mean_ctx = decode_device_timed(llm, random_prompts(batch, T, vocab, 100), steps, warmup,
                                                          vocab, whole_batch_prefill=False)
            if arch == "sominex":
                step_bytes = sizes["weight_bytes"] + batch * (sizes["state_bytes"] + sizes["kv_bytes"](mean_ctx))
            else:
                step_bytes = sizes["weight_bytes"] + batch * mean_ctx * sizes["kv_bytes_per_token"]
            gbs = step_bytes / (sec / steps) / 1e9
            row[arch] = dict(
                active_parameters_per_layer_m=round(sizes["layer_params"] / layers / 1e6, 1),
                prefill_tokens_per_s=round(T / (ms / 1e3)), prefill_ms=round(ms, 3), prefill_plain_ms=round(plain, 3),
                prefill_frac_of_tensor_peak=round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
                decode_tokens_per_s=round(batch * steps / sec), decode_ms_per_step=round(sec / steps * 1e3, 4),
                decode_launches_per_step=per_step, decode_step_mb=round(step_bytes / 1e6, 1), decode_gbs=round(gbs),
                decode_frac_of_copy_bandwidth=round(gbs / pk["hbm_gbs"], 3))
            del llm
            torch.cuda.empty_cache()
        rows[name] = row
    print(json.dumps({"metric": "prefill and decode tokens/s of Sominex beside Qwen3 at equal sizes (random weights)",
                      "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "impl": "ours",
                      "config": {"layers": layers, "vocab": vocab, "prompt_tokens": T, "decode_batch": batch,
                                 "decode_context_from": T + warmup, "decode_steps": steps, "peaks": pk["source"],
                                 "l2": "inputs larger than L2 (weights, states and cache read every step)"},
                      "sizes": rows, "clocks": clocks.stop()}))
    return 0


# ---- Mopitar beside Sominex at equal sizes ------------------------------------------------------
def mopitar_config(width, layers, vocab) -> dict:
    """Two maps behind a window, the two-branch mixer, capped attention in turn; the second capped attention
    borrows the first one's keys and values; dense and routed feed-forwards in turn."""
    H = width // 128
    G = max(H // 4, 1)
    out, lender = [], None
    dense = dict(kind="dense", ff=9 * width // 2)
    routed = dict(kind="moe", expert=dict(ff=3 * width // 4), shared=dict(ff=3 * width // 2),
                  router=dict(experts=16, top=2, groups=dict(count=4, keep=2)))
    for i in range(layers):
        mlp = routed if i % 2 else dense
        if i % 3 == 0:
            scaling = dict(factor=4.0, original=2048, fast=32.0, slow=1.0)
            out.append(dict(type="attention_2", mlp=mlp,
                            mixer=dict(heads=H, kv_heads=G, dim=128, vdim=128, scale=128 ** -0.5, diff=0.5,
                                       mask=dict(size=512, keep_first=8), rot=dict(dims=64, base=1e6, scaling=scaling))))
        elif i % 3 == 1:
            left = dict(heads=max(H // 2, 1), kv_heads=max(G // 2, 1), dim=128, vdim=128, scale=0.09, softcap=40.0,
                        rot=dict(dims=128, base=5e5))
            right = dict(inner=2 * width, state=16, dt_rank=max(width // 16, 8), conv=4)
            out.append(dict(type="parallel", mlp=mlp, mixer=dict(left=left, right=right, left_scale=1.0, right_scale=1.0)))
        else:
            m = dict(heads=H, kv_heads=G, dim=128, vdim=128, scale=128 ** -0.5, softcap=20.0, rot=dict(dims=128, base=1e4))
            if lender is not None:
                m["kv_from"] = lender
            else:
                lender = i
            out.append(dict(type="attention", mlp=mlp, mixer=m))
    return dict(architecture="Mopitar", width=width, vocab=vocab, norm=dict(eps=1e-6), layers=out)


def mopitar_bytes_and_flops(cfg: dict, T: int) -> dict:
    """Parameters a token's step multiplies by, the bytes a decode step of a batch reads at least (every matrix
    once, every state read and written, every visible key and value once), and the (query, key) pairs of a
    prompt of T tokens."""
    W, V = cfg["width"], cfg["vocab"]
    active = total = state_bytes = 0
    seen = []                      # (bytes per visible token, window, kept) of every layer that reads keys
    pair_flops = 0.0
    for layer in cfg["layers"]:
        m, mlp = layer["mixer"], layer["mlp"]
        if layer["type"] == "attention_2":
            H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mix = W * (2 * H * D + 2 * G * D + G * Vd + H * Vd)
            w, k = m["mask"]["size"], m["mask"]["keep_first"]
            seen.append((2 * (2 * G * D + G * Vd), w, k))
            pairs = sum(min(t + 1, w) + min(k, max(0, t + 1 - w)) for t in range(T))
            pair_flops += 2 * (2.0 * H * D + 2.0 * H * Vd) * pairs
        elif layer["type"] == "attention":
            H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mix = W * (H * D + H * Vd) + (0 if m.get("kv_from") is not None else W * (G * D + G * Vd))
            seen.append((2 * (G * D + G * Vd), 0, 0))
            pair_flops += (2.0 * H * D + 2.0 * H * Vd) * T * (T + 1) / 2
        else:
            l, r = m["left"], m["right"]
            H, G, D, Vd = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            mix = W * (H * D + G * D + G * Vd + H + H * Vd)
            seen.append((2 * (G * D + G * Vd), 0, 0))
            pair_flops += (2.0 * H * D + 2.0 * H * Vd) * T * (T + 1) / 2
            inner, N, R = r["inner"], r["state"], r["dt_rank"]
            mix += W * 2 * inner + inner * (R + 2 * N) + R * inner + inner * W
            state_bytes += 2 * 4 * inner * N
        if mlp["kind"] == "dense":
            a = t = 2 * W * mlp["ff"]
        else:
            r = mlp["router"]
            a = W * r["experts"] + 3 * W * (mlp["expert"]["ff"] * r["top"] + mlp["shared"]["ff"])
            t = W * r["experts"] + 3 * W * (mlp["expert"]["ff"] * r["experts"] + mlp["shared"]["ff"])
        active += mix + a
        total += mix + t

    def kv_bytes(ctx: float) -> float:
        return sum(b * (ctx if not w else min(ctx, w) + min(k, max(0.0, ctx - w))) for b, w, k in seen)
    return dict(layer_params=active, total_params=total, weight_bytes=2 * (total + 2 * V * W), state_bytes=state_bytes,
                kv_bytes=kv_bytes, pair_flops=pair_flops)


def mopitar_comparison(a, pk) -> int:
    import torch
    from gguf2bin_b200.api import LLM
    layers, vocab, batch, T = a.layers or 6, 151936, a.batch or 8, a.prefill_tokens
    steps, warmup = a.steps or 128, max(a.warmup, 8)
    max_tokens = batch * (T + warmup + steps + 128)
    rows = {}
    clocks = ClockSampler()
    clocks.start()
    for name, (width, att, ssm, mls, ff, moe, *_rest) in SOMINEX_SIZES.items():
        if a.sizes_only and name not in a.sizes_only.split(","):
            continue
        row = {}
        for arch in ("mopitar", "sominex"):
            if arch == "mopitar":
                cfg = mopitar_config(width, layers, vocab)
                sizes = mopitar_bytes_and_flops(cfg, T)
            else:
                cfg = sominex_config(width, att, ssm, mls, ff, moe, layers, vocab)
                sizes = sominex_bytes_and_flops(cfg, T)
            flops = 2.0 * T * sizes["layer_params"] + sizes["pair_flops"] + 2.0 * vocab * width
            llm = LLM.random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_seqs=batch + 1)
            first, ms, plain = timed_prompt_step(llm, random_prompts(1, T, vocab, 1), repeats=3)
            sec, per_step, mean_ctx = decode_device_timed(llm, random_prompts(batch, T, vocab, 100), steps, warmup,
                                                          vocab, whole_batch_prefill=False)
            step_bytes = sizes["weight_bytes"] + batch * (sizes["state_bytes"] + sizes["kv_bytes"](mean_ctx))
            gbs = step_bytes / (sec / steps) / 1e9
            row[arch] = dict(
                active_parameters_per_layer_m=round(sizes["layer_params"] / layers / 1e6, 1),
                prefill_tokens_per_s=round(T / (ms / 1e3)), prefill_ms=round(ms, 3), prefill_plain_ms=round(plain, 3),
                prefill_frac_of_tensor_peak=round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
                decode_tokens_per_s=round(batch * steps / sec), decode_ms_per_step=round(sec / steps * 1e3, 4),
                decode_launches_per_step=per_step, decode_step_mb=round(step_bytes / 1e6, 1), decode_gbs=round(gbs),
                decode_frac_of_copy_bandwidth=round(gbs / pk["hbm_gbs"], 3))
            del llm
            torch.cuda.empty_cache()
        rows[name] = row
    print(json.dumps({"metric": "prefill and decode tokens/s of Mopitar beside Sominex at equal sizes (random weights)",
                      "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "impl": "ours",
                      "config": {"layers": layers, "vocab": vocab, "prompt_tokens": T, "decode_batch": batch,
                                 "decode_context_from": T + warmup, "decode_steps": steps, "peaks": pk["source"],
                                 "l2": "inputs larger than L2 (weights, states and cache read every step)"},
                      "sizes": rows, "clocks": clocks.stop()}))
    return 0


WORKLOADS = {
    # name: (sizes, batch, what it is)
    "decode": ("0.6b", 8, "every sequence prefilled to half the context, then decoded"),
    "ragged8": ("8b", 8, "8 prompts with lengths uniform in [128, 2048] in ONE prompt step, then 256 decode steps"),
    "b64": ("14b", 64, "64 prompts of 512 tokens in one prompt step, decoded to a context of 2048"),
    "senotar": (None, 8, "Senotar beside Qwen3 at equal sizes: a 2,048-token prompt step and batch-8 decode steps each"),
    "levolix": (None, 8, "Levolix beside Qwen3 at equal sizes: a 2,048-token prompt step and batch-8 decode steps each"),
    "sominex": (None, 8, "Sominex beside Qwen3 at equal sizes: a 2,048-token prompt step and batch-8 decode steps each"),
    "mopitar": (None, 8, "Mopitar beside Sominex at equal sizes: a 2,048-token prompt step and batch-8 decode steps each"),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="decode steps timed (default: 512; the workload's own for ragged8 and b64)")
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=sorted(WORKLOADS),
                    help="decode: the default run; ragged8 / b64: the two larger configurations' own workloads")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has")
    ap.add_argument("--sizes", default=None, choices=["0.6b"] + sorted(OTHER_SIZES),
                    help="layer sizes: Qwen3-0.6B, or those of Qwen3-8B / 14B (default: the workload's)")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the prompt of the prefill figure (decode workload; default 2048)")
    ap.add_argument("--sizes-only", default=None,
                    help="senotar, levolix, sominex and mopitar workloads: a comma-separated subset of " + ",".join(EQUAL_SIZES))
    a = ap.parse_args()

    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "AnonymoDGH/gguf2bin is a C99 Makefile project without setup.py or "
                          "pyproject.toml, so pip cannot install it into baseline/_ref; it has no "
                          "GPU code and no batching"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.warmup < 3:
        a.warmup = 3
    if a.workload == "senotar":
        return senotar_comparison(a, peaks())
    if a.workload == "levolix":
        return levolix_comparison(a, peaks())
    if a.workload == "sominex":
        return sominex_comparison(a, peaks())
    if a.workload == "mopitar":
        return mopitar_comparison(a, peaks())

    import numpy as np
    import torch
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.api import LLM

    w_sizes, w_batch, w_what = WORKLOADS[a.workload]
    a.sizes = a.sizes or w_sizes
    a.batch = a.batch or w_batch
    cfg = dict(QWEN3_0P6B)
    cfg.update(OTHER_SIZES.get(a.sizes, {}))
    full_layers = cfg["num_hidden_layers"]
    if a.layers is None:
        a.layers = full_layers
    cfg["num_hidden_layers"] = a.layers
    name = {"0.6b": "Qwen3-0.6B", "8b": "Qwen3-8B", "14b": "Qwen3-14B"}[a.sizes]
    pk = peaks()
    sizes = model_bytes_and_flops(cfg, a.layers)
    vocab = cfg["vocab_size"]

    # ---- the workload's prompts and steps ----------------------------------------------------
    if a.workload == "decode":
        start_ctx = a.context // 2
        steps = min(a.steps or 512, a.context - start_ctx - 1)
        decode_prompts = random_prompts(a.batch, start_ctx - a.warmup, vocab, 100)
        prefill_prompts = random_prompts(1, a.prefill_tokens, vocab, 1)
        seq_len = a.context
        points_wanted = not a.no_points
        max_batch = max(64 if points_wanted else a.batch, a.batch)
        max_tokens = max(max_batch * (a.context + 64), a.prefill_tokens + 64)
    elif a.workload == "ragged8":
        lengths = np.random.default_rng(2024).integers(128, 2049, a.batch).tolist()
        steps = a.steps or 256
        decode_prompts = [random_prompts(1, n, vocab, 300 + i)[0] for i, n in enumerate(lengths)]
        prefill_prompts = decode_prompts
        seq_len = max(lengths) + a.warmup + steps
        points_wanted, max_batch = False, a.batch
        max_tokens = sum(-(-(n + a.warmup + steps + 2) // 64) * 64 for n in lengths) + 64
    else:
        a.context = 2048
        steps = min(a.steps or 10 ** 9, a.context - 512 - a.warmup)
        decode_prompts = random_prompts(a.batch, 512, vocab, 500)
        prefill_prompts = decode_prompts
        seq_len = a.context
        points_wanted, max_batch = False, a.batch
        max_tokens = a.batch * (a.context + 64)

    free0, total_mem = torch.cuda.mem_get_info()
    llm = LLM.random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_seqs=max_batch + 1)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()

    # ---- prefill: one step over the prompts, logits at each last place ------------------------
    pre_first, pre, pre_plain = timed_prompt_step(llm, prefill_prompts, repeats=3)
    pre_lengths = [len(p) for p in prefill_prompts]
    pre_tokens = sum(pre_lengths)
    pre_flops = prefill_flops(cfg, a.layers, pre_lengths)
    prefill = dict(value=pre_tokens / (pre / 1e3), tokens=pre_tokens, ms=pre,
                   frac=pre_flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12),
                   first_ms=pre_first, plain_ms=pre_plain, sequences=len(pre_lengths))

    # ---- decode, device-timed -----------------------------------------------------------------
    clocks = ClockSampler()
    clocks.start()
    sec, per_step, mean_ctx = decode_device_timed(llm, decode_prompts, steps, a.warmup, vocab,
                                                  whole_batch_prefill=a.workload != "decode")
    clock_info = clocks.stop()
    value = a.batch * steps / sec
    roofline = hbm_roofline(sizes, a.batch, mean_ctx, sec / steps, pk)

    # ---- decode through the Python entry point, host tokens in and out -------------------------
    e2e_steps = min(steps, 256)
    e2e_prompts = [p + [1] * a.warmup for p in decode_prompts]     # the same lengths as the timed steps start from
    llm.generate(e2e_prompts[:1], n=4, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                 ignore_eos=True)
    e2e_runs = []                      # three whole calls; the median is reported, all are listed
    for _ in range(3):
        llm.generate(e2e_prompts, n=e2e_steps + 1, temperature=0.0, top_k=0, top_p=1.0,
                     repeat_penalty=1.0, ignore_eos=True, max_batch=a.batch)
        acct = llm.last_decode
        e2e_runs.append((acct["tokens"] / acct["seconds"], acct["steps"]))
    e2e_value, e2e_count = sorted(e2e_runs)[1]
    # the same call with the entry point's own sampling parameters (temperature 0.7, top-k 40,
    # top-p 0.9, repeat penalty 1.1: what a user who sets nothing gets); the second of two calls
    sampled = []
    for _ in range(2):
        llm.generate(e2e_prompts, n=e2e_steps + 1, ignore_eos=True, max_batch=a.batch)
        sampled.append(llm.last_decode["tokens"] / llm.last_decode["seconds"])
    e2e = dict(value=e2e_value, unit="tokens/s", h2d_bytes_per_step=4 * a.batch,
               d2h_bytes_per_step=4 * a.batch, steps=e2e_count,
               runs=[round(v, 1) for v, _ in e2e_runs], default_sampling=round(sampled[-1], 1),
               graphs_captured=llm.engine.graph_captures)

    # ---- other batch sizes ------------------------------------------------------------------------
    points = {}
    if points_wanted:
        room = a.context - start_ctx - 1
        for b, k in ((1, min(room, 256)), (64, min(room, 128))):    # their own step counts, whatever --steps says:
            warm = max(a.warmup, 16)                                # twenty steps of 0.7 ms mostly measure the clocks settling
            s, _, ctx_b = decode_device_timed(llm, random_prompts(b, start_ctx - warm, vocab, 100), k,
                                              warm, vocab, whole_batch_prefill=False)
            r = hbm_roofline(sizes, b, ctx_b, s / k, pk)
            points[f"decode_b{b}"] = b * k / s
            points[f"decode_b{b}_ms_per_step"] = s / k * 1e3
            points[f"decode_b{b}_gbs"] = r["achieved"]
            points[f"decode_b{b}_frac"] = r["frac"]

    first_ctx = mean_ctx - steps / 2.0
    out = {
        "metric": f"decode tokens/s ({name} sizes, random weights, batch {a.batch}, "
                  f"context {first_ctx:.0f}->{first_ctx + steps:.0f})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": a.warmup,
        "ms_per_step": sec / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"{name} sizes, random weights", "workload": f"{a.workload}: {w_what}",
                   "global_batch": a.batch,
                   "seq_len": seq_len, "decode_from": round(first_ctx, 1), "layers": a.layers,
                   "layers_of_config": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": vocab, "tied": bool(cfg["tie_word_embeddings"]), "parallelism": "none (1 GPU)",
                   "l2": "inputs larger than L2 (weights + cache read every step)",
                   "sampling": "greedy on device",
                   "weights": "made on the device (Philox normal), never on disk",
                   "device_gb_free_before_after": f"{free0 / 1e9:.1f} -> {free1 / 1e9:.1f} of {total_mem / 1e9:.1f}"},
        "e2e": e2e, "gpu_launches": per_step * steps, "launches_per_step": per_step,
        "prefill": prefill, "roofline": roofline, "points": points, "clocks": clock_info,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
