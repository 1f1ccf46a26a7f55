#!/usr/bin/env python3
"""Throughput of the engine at Qwen3-8B layer sizes with random weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--batch 8] [--layers L] [--prompt-len 2048] [--context 4096]

A "step" is one decode step of a batch of sequences that were prefilled to --prompt-len tokens.
`value` is decoded tokens per second of K steps timed on the device (CUDA events, after W warm-up
steps); every step reads all weights (about 15 GB, far larger than the 126 MB L2), so no flush is
needed between steps.  `e2e` is the same through the Python entry point with host tokens in and
out of every step, over at least 64 steps that follow an untimed round (which holds the capture of
the step's CUDA graph).  `prefill` times one 2,048-token prompt through `Engine.step` (host packing
and upload included); `points` holds decode at batch 1 and 64 and, unless --no-workloads, the two
other workloads the baseline names, run through `generate` and timed by its own statistics on the
host: 16 unequal prompts of 32 to 1,024 tokens with 256 decode steps at Qwen3-0.6B sizes, and 8
prompts of 1,024 tokens with 128 decode steps at Qwen3-32B sizes.  `fp32_check` compares the
bfloat16 engine with the true 32-bit engine on the same full-size model (a 64-token prompt).
One JSON line goes to standard output.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960,
                tie_word_embeddings=False, eos_token_id=151645)
# The other two sizes the reference architecture is usually quoted at (same layer formulas).
SIZES = {
    "8b": {},
    "0.6b": dict(hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=3072, tie_word_embeddings=True),
    "32b": dict(hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                intermediate_size=25600),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.time(), line.strip()))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows) -> dict:
        sm, mx, reasons = [], [], set()
        for ts, line in self.rows:
            if not any(a <= ts <= b for a, b in windows):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm() -> int:
    # The reference is a Rust workspace (Cargo.toml, no setup.py / pyproject.toml): pip cannot
    # install it, there is no Rust toolchain in this image, and its GPU backends need Vulkan or Metal.
    print(json.dumps({"impl": "reference", "unavailable":
                      "xigh/herbert-rs is a Rust workspace with Vulkan/Metal GPU backends: no Python package to install offline, no cargo/rustc in the image, no graphics stack on the box"}))
    return 0


WORKLOADS = {
    # the baseline's fourth and fifth configurations (Qwen3-0.6B and Qwen3-32B layer sizes), as written there
    "0.6b": dict(size="0.6b", prompts=16, min_len=32, max_len=1024, steps=256),
    "32b": dict(size="32b", prompts=8, min_len=1024, max_len=1024, steps=128),
}


def run_workload(name: str, windows: list) -> dict:
    """One of the baseline's other workloads through the public `generate`: decode tokens per second
    by the loop's own statistics (host clock around the decode steps, tokens read back every step)."""
    import numpy as np
    import torch

    import herbert_rs_b200 as hb

    w = WORKLOADS[name]
    cfg = dict(QWEN3_8B)
    cfg.update(SIZES[w["size"]])
    rng = np.random.default_rng(1)
    lens = [int(n) for n in rng.integers(w["min_len"], w["max_len"] + 1, w["prompts"])]
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lens]
    rt = hb.Runtime("cuda", torch.bfloat16)
    model = hb.random_model(cfg, 0, rt)
    per_seq = max(lens) + w["steps"] + 1
    engine = hb.Engine(model, max_tokens=hb.Engine.pages_for(per_seq, w["prompts"]) * rt.page_size, max_slots=w["prompts"])
    opt = hb.GenerationOptions(max_tokens=w["steps"] + 1, ignore_eos=True)      # the first token comes from the prompts' step
    greedy = hb.SamplingParams(temperature=0.0)
    hb.generate(engine, prompts, hb.GenerationOptions(max_tokens=12, ignore_eos=True), greedy)    # untimed: graph capture, workspace growth
    torch.cuda.synchronize()
    t0 = time.time()
    res = hb.generate(engine, prompts, opt, greedy)
    windows.append((t0, time.time()))
    st = res.stats
    out = {"decode_tok_s": round(st.decode_tokens_per_second, 1), "prefill_tok_s": round(st.prefill_tokens_per_second, 1),
           "decode_steps": st.decode_steps, "prompt_tokens": st.prompt_tokens, "ms_per_step": round(st.decode_seconds / max(1, st.decode_steps) * 1e3, 4),
           "layers": cfg["num_hidden_layers"], "prompts": w["prompts"]}
    del engine, model
    torch.cuda.empty_cache()
    return out


def fp32_check(cfg: dict, bf16_engine, n_tokens: int = 64) -> dict:
    """The bfloat16 engine against the true 32-bit engine on the same model (same seed, same
    weights: bfloat16 values widened exactly) at full size: logits at every position of a prompt."""
    import numpy as np
    import torch

    import herbert_rs_b200 as hb

    ids = np.random.default_rng(7).integers(0, cfg["vocab_size"], n_tokens).tolist()
    s = bf16_engine.alloc_slot()
    low = bf16_engine.step([(s, ids)], "all").double().cpu()
    bf16_engine.free_slot(s)
    rt = hb.Runtime("cuda", torch.float32)
    eng = hb.Engine(hb.random_model(cfg, 0, rt), max_tokens=hb.Engine.pages_for(n_tokens) * rt.page_size, max_slots=1)
    s = eng.alloc_slot()
    ref = eng.step([(s, ids)], "all").double().cpu()
    eng.free_slot(s)
    eng.check_kernels()
    del eng
    torch.cuda.empty_cache()
    top2 = ref.topk(2, dim=-1).values
    gap = top2[:, 0] - top2[:, 1]
    differ = low.argmax(-1) != ref.argmax(-1)
    # where the two engines choose another token, how far apart the 32-bit engine's two best logits were there,
    # and how much lower it rates the bfloat16 engine's choice: both small against max_abs_err if the choice was a near-tie
    lost = (ref.max(-1).values - ref.gather(1, low.argmax(-1, keepdim=True))[:, 0])
    return {"tokens": n_tokens, "layers": cfg["num_hidden_layers"], "max_abs_err": round(float((low - ref).abs().max()), 5),
            "logit_std": round(float(ref.std()), 4), "argmax_agree": round(float((~differ).double().mean()), 4),
            "median_top2_gap": round(float(gap.median()), 5),
            "largest_gap_where_they_differ": round(float(gap[differ].max()) if bool(differ.any()) else 0.0, 5),
            "largest_logit_given_up": round(float(lost.max()), 5)}


# ---- the Kebisun design beside the dense decoder at equal sizes ---------------------------------------
def _kebisun_config(width, heads, dim, rot, vdim, kv_rank, q_rank, window, gla_heads, gla_dk, gla_dv, ff, experts, top, expert_ff,
                    vocab, decay_rank=32):
    latent = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
              "scale": (dim + rot) ** -0.5, "mask": {"size": window},
              "rot": {"base": 10000.0, "dims": rot, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    gla = {"heads": gla_heads, "dim": gla_dk, "vdim": gla_dv, "tau": 16.0, "decay_rank": decay_rank}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}}
    layers = [{"type": "latent_attention", "mixer": latent, "mlp": dense}, {"type": "gla", "mixer": gla, "mlp": moe},
              {"type": "latent_attention", "mixer": latent, "mlp": moe}, {"type": "gla", "mixer": gla, "mlp": dense}]
    return {"architecture": "Kebisun", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": layers}


def _votapel_config(width, heads, kv_heads, dim, experts, top, groups, keep, expert_ff, shared_ff, vocab, layers=4,
                    max_positions=8192):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 30.0,
             "q_temp": {"coef": 0.1, "every": 1024}}
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "shared": {"ff": shared_ff},
           "router": {"experts": experts, "top": top, "scale": 1.0, "groups": {"count": groups, "keep": keep}}}
    return {"architecture": "Votapel", "vocab": vocab, "width": width, "max_positions": max_positions, "norm": {"eps": 1e-6},
            "residual_mult": 0.5, "layers": [{"type": "attention", "mixer": mixer, "mlp": moe} for _ in range(layers)]}


def _begupel_config(width, heads, kv_heads, dim, vdim, window, scan_heads, scan_qk_heads, scan_dk, scan_dv, ff, vocab,
                    buckets=65536, taps=4, groups=4):
    lightning = {"heads": scan_heads, "dim": scan_dk, "vdim": scan_dv,
                 "decay": [round(1.0 - 2.0 ** -(5 + 3 * h / max(1, scan_heads - 1)), 6) for h in range(scan_heads)]}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "mask": {"size": window},
            "rot": {"base": 10000.0, "dims": dim // 2, "scaling": {"factor": 4.0}}}
    right = {"heads": scan_heads, "kv_heads": scan_qk_heads, "dim": scan_dk, "vdim": scan_dv, "conv": taps}
    side = {"left": left, "right": right, "left_scale": 0.5, "right_scale": 0.5}
    dense = {"kind": "dense", "ff": ff}
    layers = [{"type": "lightning", "mixer": lightning, "mlp": dense}, {"type": "parallel", "mixer": side, "mlp": dense},
              {"type": "lightning", "mixer": lightning, "mlp": dense}, {"type": "parallel", "mixer": side, "mlp": dense}]
    return {"architecture": "Begupel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6, "groups": groups},
            "canon": {"taps": taps}, "logit_softcap": 30.0,
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": 1000003, "mul_cur": 31}}, "layers": layers}


def _nefivik_config(width, heads, kv_heads, dim, vdim, window, delta_heads, delta_dim, experts, top, groups, keep, expert_ff,
                    side, vocab, taps=4):
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "mask": {"size": window}, "conv": taps,
           "rot": {"base": 10000.0, "dims": dim // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    delta = {"heads": delta_heads, "dim": delta_dim}
    moe = {"kind": "moe", "expert": {"ff": expert_ff, "limit": 7.0},
           "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}
    layers = [{"type": "attention", "mixer": att, "mlp": moe}, {"type": "general_delta", "mixer": delta, "mlp": moe},
              {"type": "attention", "mixer": dict(att, kv_from=0), "mlp": moe}, {"type": "general_delta", "mixer": delta, "mlp": moe}]
    return {"architecture": "Nefivik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "token_side": {"dim": side},
            "layers": layers}


NEFIVIK_SIZES = {
    # Nefivik layer sizes (two layers of windowed sigmoid attention, the second reading the first one's keys and values, two of
    # the generalised delta rule, routed experts in every layer); beside them Begupel (the closest design in its mixers:
    # windowed attention behind a convolution beside a delta rule, a norm on every sublayer's result), Votapel (the closest
    # in its feed-forward: gated experts chosen within groups) and the dense decoder, each of the same width, depth, heads
    # and head size
    "1k": (dict(width=1024, heads=8, kv_heads=4, dim=128, vdim=128, window=4096, delta_heads=8, delta_dim=128, experts=16, top=2,
                groups=4, keep=2, expert_ff=768, side=64, vocab=32000), "1k"),
    "2k": (dict(width=2048, heads=16, kv_heads=8, dim=128, vdim=128, window=4096, delta_heads=16, delta_dim=128, experts=32, top=4,
                groups=8, keep=4, expert_ff=1408, side=128, vocab=32000), "2k"),
}

BEGUPEL_SIZES = {
    # Begupel layer sizes (two lightning layers, two with windowed attention beside a gated delta rule); beside them
    # Kebisun with recurrent heads of the same number and sizes (the closest design: a scan over a matrix state, a
    # windowed attention, a norm on every sublayer's result) and the dense decoder of the same width, depth, heads,
    # head size and feed-forward width
    "1k": (dict(width=1024, heads=8, kv_heads=4, dim=128, vdim=128, window=4096, scan_heads=8, scan_qk_heads=4, scan_dk=128,
                scan_dv=128, ff=3072, vocab=32000),
           dict(width=1024, heads=8, dim=64, rot=32, vdim=64, kv_rank=256, q_rank=384, window=4096, gla_heads=8, gla_dk=128,
                gla_dv=128, ff=3072, experts=16, top=2, expert_ff=768, vocab=32000),
           dict(hidden_size=1024, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=4, head_dim=128,
                intermediate_size=3072, vocab_size=32000, eos_token_id=31999)),
    "2k": (dict(width=2048, heads=16, kv_heads=8, dim=128, vdim=128, window=4096, scan_heads=16, scan_qk_heads=8, scan_dk=128,
                scan_dv=128, ff=8192, vocab=32000),
           dict(width=2048, heads=16, dim=128, rot=64, vdim=128, kv_rank=512, q_rank=768, window=4096, gla_heads=16, gla_dk=128,
                gla_dv=128, ff=8192, experts=32, top=4, expert_ff=1408, vocab=32000),
           dict(hidden_size=2048, num_hidden_layers=4, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                intermediate_size=8192, vocab_size=32000, eos_token_id=31999)),
}

VOTAPEL_SIZES = {
    # Votapel layer sizes, and the dense decoder of the same width, depth, heads and head size beside them; a token's
    # experts and the shared one together are as wide as the dense feed-forward
    "1k": (dict(width=1024, heads=16, kv_heads=8, dim=64, experts=16, top=2, groups=4, keep=2, expert_ff=768, shared_ff=1536,
                vocab=32000),
           dict(hidden_size=1024, num_hidden_layers=4, num_attention_heads=16, num_key_value_heads=8, head_dim=64,
                intermediate_size=3072, vocab_size=32000, eos_token_id=31999)),
    "2k": (dict(width=2048, heads=16, kv_heads=8, dim=128, experts=32, top=4, groups=8, keep=4, expert_ff=1408, shared_ff=2560,
                vocab=32000),
           dict(hidden_size=2048, num_hidden_layers=4, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                intermediate_size=8192, vocab_size=32000, eos_token_id=31999)),
}

DESIGN_SIZES = {
    # Kebisun layer sizes, and the dense decoder of the same width, depth and feed-forward width beside them
    "1k": (dict(width=1024, heads=8, dim=64, rot=32, vdim=64, kv_rank=256, q_rank=384, window=4096, gla_heads=4, gla_dk=128,
                gla_dv=256, ff=3072, experts=16, top=2, expert_ff=768, vocab=32000),
           dict(hidden_size=1024, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=4, head_dim=128,
                intermediate_size=3072, vocab_size=32000, eos_token_id=31999)),
    "2k": (dict(width=2048, heads=16, dim=128, rot=64, vdim=128, kv_rank=512, q_rank=768, window=4096, gla_heads=4, gla_dk=256,
                gla_dv=512, ff=8192, experts=32, top=4, expert_ff=1408, vocab=32000),
           dict(hidden_size=2048, num_hidden_layers=4, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                intermediate_size=8192, vocab_size=32000, eos_token_id=31999)),
}


def _launcher_work(name, n, ctx):
    """(FLOPs, bytes) that all `n` launches of a launcher do in one step of `ctx` (a dict of the step's
    and the model's sizes), for the launchers compared between the two models; None for the others."""
    T, L, B = ctx["tokens"], ctx["kv_len"], ctx["seqs"]
    pairs = T * (L - (T // B - 1) / 2.0) if T > B else T * L        # (query, key) pairs per head: causal prompt / one query over L keys
    es = 2
    if ctx["kind"] == "kebisun":
        H, rk, dr, dn, dv, D = ctx["heads"], ctx["kv_rank"], ctx["rot"], ctx["dim"], ctx["vdim"], ctx["width"]
        if name in ("hb_latent_attention", "hb_latent_attention_mma_bf16"):
            return n * 2.0 * pairs * H * (2 * rk + dr), n * (B * L * (rk + dr) * es + T * H * (2 * rk + dr) * 4)
        if name == "hb_headwise_gemm":      # two per latent layer: dn -> rk and rk -> dv
            per = n / 2.0
            return per * 2.0 * T * H * rk * (dn + dv), per * (H * rk * (dn + dv) * es + T * H * (rk + dn + dr + rk + dv) * 4)
        if name == "hb_layernorm_residual":
            return n * 8.0 * T * D, n * T * D * (4 + 4 + 4 + es)
        if name == "hb_gla_scan":
            gh, dk, gv = ctx["gla_heads"], ctx["gla_dk"], ctx["gla_dv"]
            return n * 4.0 * T * gh * dk * gv, n * (T * gh * (3 * dk + 2 * gv) * 4 + 2 * B * gh * dk * gv * 4)
        if name in ("hb_moe_experts", "hb_moe_experts_grouped_bf16"):
            E, top, F = ctx["experts"], ctx["top"], ctx["expert_ff"]
            return n * 4.0 * T * top * F * D, n * (min(E, T * top) * 2 * F * D * es + T * D * (es + 4))
    elif ctx["kind"] == "votapel":
        H, KV, hd, D = ctx["heads"], ctx["kv_heads"], ctx["dim"], ctx["width"]
        if name in ("hb_attention_prefill_tc_bf16", "hb_attention_prefill_bf16", "hb_attention_decode_bf16", "hb_attention_simt"):
            return n * 4.0 * pairs * H * hd, n * (B * L * KV * hd * es + 2 * T * H * hd * es)      # one plane: the values are the keys
        if name == "hb_scaled_residual_norm":
            return n * 6.0 * T * D, n * T * D * (4 + 4 + 4 + es)
        if name == "hb_qk_prepare_cache":
            return n * 2.0 * T * (H + KV) * hd, n * T * (H + KV) * hd * (4 + es)
        if name in ("hb_moe_experts", "hb_moe_experts_grouped_bf16", "hb_moe_experts_tc_bf16"):
            E, top, F = ctx["experts"], ctx["top"], ctx["expert_ff"]
            return n * 6.0 * T * top * F * D, n * (min(E, T * top) * 3 * F * D * es + T * D * (es + 4))
        if name == "hb_moe_route":
            return n * 2.0 * T * ctx["experts"] * D, n * (T * D * es + ctx["experts"] * D * es)
    elif ctx["kind"] == "begupel":
        H, KV, D = ctx["heads"], ctx["kv_heads"], ctx["width"]
        hd = max(ctx["dim"], ctx["vdim"])
        sh, sg, dk, dv = ctx["scan_heads"], ctx["scan_qk_heads"], ctx["scan_dk"], ctx["scan_dv"]
        if name in ("hb_attention_prefill_tc_bf16", "hb_attention_prefill_bf16", "hb_attention_decode_bf16", "hb_attention_simt"):
            return n * 4.0 * pairs * H * hd, n * (2 * B * L * KV * hd * es + 2 * T * H * hd * es)
        if name == "hb_linear_scan":
            # half of the launches decay and add an outer product (4 operations a state entry), half run the delta
            # rule (7); every launch reads q, k, v and writes o as floats and reads and writes every sequence's state
            half = n / 2.0
            rows = T * sh * (2 * dk + 2 * dv) * 4 + T * (2 * sg * dk + 2 * sh * dv + 2 * sh) * 4
            return half * (4.0 + 7.0) * T * sh * dk * dv, half * rows + n * 2 * B * sh * dk * dv * 4
        if name == "hb_group_rmsnorm_residual":
            return n * 6.0 * T * D, n * T * D * (4 + 4 + 4 + es)
        if name == "hb_short_conv":       # the stream's rows (D channels, every layer) and the delta rule's q, k, v rows
            per = n / 6.0
            C = 2 * sg * dk + sh * dv
            return n * 8.0 * T * D, per * (4 * T * D * (4 + es) + 2 * T * C * 8)
        if name == "hb_qkv_rotary_cache":
            return n * 6.0 * T * (H + 2 * KV) * hd, n * T * ((H + 2 * KV) * hd * (4 + es))
        if name == "hb_gated_rmsnorm":
            return n * 8.0 * T * sh * dv, n * T * sh * dv * (4 + 4 + es)
    elif ctx["kind"] == "nefivik":
        H, KV, D = ctx["heads"], ctx["kv_heads"], ctx["width"]
        hd = max(ctx["dim"], ctx["vdim"])
        dh, dn = ctx["delta_heads"], ctx["delta_dim"]
        if name in ("hb_attention_prefill_tc_bf16", "hb_attention_prefill_bf16", "hb_attention_decode_bf16", "hb_attention_simt"):
            return n * 4.0 * pairs * H * hd, n * (2 * B * L * KV * hd * es + 2 * T * H * hd * es)
        if name == "hb_general_delta_scan":
            # 9 operations a state entry and token; a launch reads five key-side vectors and v, writes o, as floats,
            # and reads and writes every sequence's state
            return n * 9.0 * T * dh * dn * dn, n * (T * dh * dn * 7 * 4 + 2 * B * dh * dn * dn * 4)
        if name == "hb_general_delta_prepare":
            return n * 2.0 * T * dh * dn * 64, n * T * dh * dn * (3 + 5) * 4
        if name == "hb_gated_norm_residual":
            return n * 8.0 * T * D, n * T * D * (4 + 4 + 4 + 4 + es)
        if name == "hb_short_conv":       # q, k, v rows of the storing layer, q rows of the reading one
            C = (H + KV) * ctx["dim"] + KV * ctx["vdim"]
            return n * 8.0 * T * C, n / 2.0 * T * (C + H * ctx["dim"]) * 8
        if name == "hb_qkv_rotary_cache":
            return n * 6.0 * T * (H + 2 * KV) * hd, n / 2.0 * T * ((2 * H + 2 * KV) * hd * (4 + es))
        if name == "hb_gated_rmsnorm":
            return n * 8.0 * T * dh * dn, n * T * dh * dn * (4 + 4 + es)
        if name in ("hb_moe_experts", "hb_moe_experts_grouped_bf16", "hb_moe_experts_tc_bf16"):
            E, top, F = ctx["experts"], ctx["top"], ctx["expert_ff"]
            return n * 6.0 * T * top * F * D, n * (min(E, T * top) * 3 * F * D * es + T * D * (es + 4))
        if name == "hb_moe_route":
            return n * 2.0 * T * ctx["experts"] * D, n * (T * D * es + ctx["experts"] * D * es)
    else:
        H, KV, hd, D = ctx["heads"], ctx["kv_heads"], ctx["head_dim"], ctx["width"]
        if name in ("hb_attention_prefill_tc_bf16", "hb_attention_prefill_bf16", "hb_attention_decode_bf16",
                    "hb_attention_decode_fused_bf16", "hb_attention_simt"):
            return n * 4.0 * pairs * H * hd, n * (2 * B * L * KV * hd * es + 2 * T * H * hd * es)
        if name == "hb_rmsnorm":
            return n * 4.0 * T * D, n * T * D * (4 + es)
    return None


def _design_point(hb, ops, torch, np, cfg, ctx, pk, prompt_len, batch, steps, warmup, windows):
    """Prefill of one prompt and decode at `batch` for one model: tokens per second, and per launcher
    the time of a prompt step and of an eager decode step with its distance from the roofline."""
    rt = hb.Runtime("cuda", torch.bfloat16)
    model = hb.random_model(cfg, 0, rt)
    context = prompt_len + steps + warmup + 8
    engine = hb.Engine(model, max_tokens=batch * (context + 64), max_slots=batch)
    rng = np.random.default_rng(0)
    V = model.spec.vocab_size
    out = {}

    def timed_step(entries, kv_len):
        with ops.timed() as t:
            engine.step(entries, "last")
        rows = {}
        c = dict(ctx, tokens=sum(len(x) for _, x in entries), seqs=len(entries), kv_len=kv_len)
        for name, (n, ms) in t.by_kernel().items():
            row = {"launches": n, "ms": round(ms, 4)}
            work = _launcher_work(name, n, c)
            if work is not None and ms > 0:
                roof_ms = max(work[0] / (pk["bf16_tflops"] * 1e9), work[1] / (pk["hbm_gbs"] * 1e6))
                row["of_roofline"] = round(roof_ms / ms, 4)
            rows[name] = row
        return rows

    # prefill: one prompt
    s = engine.alloc_slot()
    for _ in range(max(2, warmup // 2)):
        engine.step([(s, rng.integers(0, V, prompt_len).tolist())], "last")
        engine.free_slot(s); s = engine.alloc_slot()
    ids = rng.integers(0, V, prompt_len).tolist()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(); t0 = time.time()
    e0.record(); engine.step([(s, ids)], "last"); e1.record(); torch.cuda.synchronize()
    windows.append((t0, time.time()))
    out["prefill_ms"] = round(e0.elapsed_time(e1), 3)
    out["prefill_tok_s"] = round(prompt_len / e0.elapsed_time(e1) * 1e3, 1)
    engine.free_slot(s); s = engine.alloc_slot()
    out["prefill_by_launcher"] = timed_step([(s, ids)], prompt_len)
    engine.free_slot(s)
    # decode: `batch` sequences after their prompts
    slots = [engine.alloc_slot() for _ in range(batch)]
    for sl in slots:
        engine.step([(sl, rng.integers(0, V, prompt_len).tolist())], "none")
    tok = lambda: [(sl, [int(rng.integers(0, V))]) for sl in slots]  # noqa: E731
    for _ in range(warmup):
        engine.step(tok(), "last")
    torch.cuda.synchronize(); t0 = time.time()
    e0.record()
    for _ in range(steps):
        engine.step(tok(), "last")
    e1.record(); torch.cuda.synchronize()
    windows.append((t0, time.time()))
    out["decode_ms_per_step"] = round(e0.elapsed_time(e1) / steps, 4)
    out["decode_tok_s"] = round(batch * steps / e0.elapsed_time(e1) * 1e3, 1)
    out["decode_kernels_per_step"] = engine.kernels_per_graph.get(batch)
    engine.use_graphs = False
    engine.step(tok(), "last")
    out["decode_by_launcher"] = timed_step(tok(), prompt_len + warmup + steps + 2)
    out["weight_bytes_per_step"] = model.weight_bytes(batch)
    out["decode_of_hbm_roofline"] = round(out["weight_bytes_per_step"] / (pk["hbm_gbs"] * 1e6) / out["decode_ms_per_step"], 4)
    del engine, model
    torch.cuda.empty_cache()
    return out


def run_design(args) -> int:
    """`--design begupel|kebisun|nefivik|votapel`: prefill and decode of that design at layer sizes that resemble a
    real model's, beside the dense decoder of equal width, depth and feed-forward width (random weights,
    bfloat16, four layers each); Begupel also beside Kebisun with recurrent heads of equal sizes, Nefivik also beside
    Begupel and Votapel."""
    import numpy as np
    import torch

    import herbert_rs_b200 as hb
    from herbert_rs_b200 import ops

    pk = peaks()
    sampler, windows = ClockSampler(), []
    sampler.start()
    result = {}
    table, make = {"kebisun": (DESIGN_SIZES, _kebisun_config), "votapel": (VOTAPEL_SIZES, _votapel_config),
                   "begupel": (BEGUPEL_SIZES, _begupel_config), "nefivik": (NEFIVIK_SIZES, _nefivik_config)}[args.design]
    for size in (sorted(table) if args.design_size == "all" else [args.design_size]):
        closest = None
        beside = None
        if args.design == "begupel":
            kb, closest, dense = table[size]
        elif args.design == "nefivik":
            kb, beside = table[size]
            dense = BEGUPEL_SIZES[beside][2]
        else:
            kb, dense = table[size]
        kcfg = make(**kb)
        qcfg = dict(QWEN3_8B)
        qcfg.update(dense)
        kctx = dict(kb, kind=args.design)
        qctx = dict(kind="dense", heads=dense["num_attention_heads"], kv_heads=dense["num_key_value_heads"],
                    head_dim=dense["head_dim"], width=dense["hidden_size"])
        result[size] = {
            args.design: _design_point(hb, ops, torch, np, kcfg, kctx, pk, args.prompt_len, args.batch, args.steps, args.warmup, windows),
            "dense": _design_point(hb, ops, torch, np, qcfg, qctx, pk, args.prompt_len, args.batch, args.steps, args.warmup, windows),
        }
        if closest is not None:
            result[size]["kebisun"] = _design_point(hb, ops, torch, np, _kebisun_config(**closest), dict(closest, kind="kebisun"), pk,
                                                    args.prompt_len, args.batch, args.steps, args.warmup, windows)
        if beside is not None:
            for other, sizes, maker in (("begupel", BEGUPEL_SIZES, _begupel_config), ("votapel", VOTAPEL_SIZES, _votapel_config)):
                ob = sizes[beside][0]
                result[size][other] = _design_point(hb, ops, torch, np, maker(**ob), dict(ob, kind=other), pk, args.prompt_len,
                                                    args.batch, args.steps, args.warmup, windows)
    sampler.stop()
    print(json.dumps({"metric": f"{args.design.capitalize()} and the dense decoder at equal sizes: prefill and decode tokens/s", "unit": "tokens/s",
                      "n_gpus": 1, "impl": "ours", "dtype": "bf16", "data": "synthetic", "steps": args.steps, "warmup": args.warmup,
                      "config": {"prompt_len": args.prompt_len, "batch": args.batch, "layers": 4,
                                 "timing": "CUDA events; every decode step reads all weights, a prompt step reads activations larger than L2 at the 2k size"},
                      "peaks": pk, "sizes": result, "clocks": sampler.summary(windows)}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--size", default="8b", choices=sorted(SIZES), help="layer sizes: Qwen3-8B (the headline), 0.6B or 32B")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the size has (both numbers are reported)")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 decode points")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill measurement")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end measurement")
    ap.add_argument("--no-workloads", action="store_true", help="skip the 0.6B and 32B workloads of the baseline")
    ap.add_argument("--no-fp32-check", action="store_true", help="skip the comparison with the 32-bit engine")
    ap.add_argument("--no-pdl", action="store_true", help="prompts without programmatic dependent launch")
    ap.add_argument("--pdl-graph", type=int, default=None, help="programmatic dependent launch inside recorded decode steps (0, 1, 2)")
    ap.add_argument("--workload", default=None, choices=["0.6b", "32b"],
                    help="run only this workload of the baseline and print its line")
    ap.add_argument("--design", default=None, choices=["begupel", "kebisun", "nefivik", "votapel"],
                    help="measure this design beside the dense decoder at equal sizes instead of the headline workload")
    ap.add_argument("--design-size", default="all", choices=["all"] + sorted(DESIGN_SIZES))
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (asked for {args.gpus}): this library has no multi-GPU path")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.design is not None:
        return run_design(args)
    if args.workload is not None:
        sampler, windows = ClockSampler(), []
        sampler.start()
        out = run_workload(args.workload, windows)
        sampler.stop()
        w = WORKLOADS[args.workload]
        print(json.dumps({"metric": f"Qwen3-{w['size'].upper()} decode tok/s through generate ({w['prompts']} prompts of {w['min_len']}..{w['max_len']} tokens, {w['steps']} steps)",
                          "value": out["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "impl": "ours", "dtype": "bf16",
                          "data": "synthetic", "workload": out, "clocks": sampler.summary(windows)}))
        return 0

    import numpy as np
    import torch

    import herbert_rs_b200 as hb
    from herbert_rs_b200 import ops
    from herbert_rs_b200.sampling import device_choose

    if args.no_pdl:
        ops.options.pdl_eager = False
    if args.pdl_graph is not None:
        ops.options.pdl_graph = args.pdl_graph
    pk = peaks()
    cfg = dict(QWEN3_8B)
    cfg.update(SIZES[args.size])
    layers_full = cfg["num_hidden_layers"]
    if args.layers is None:
        args.layers = layers_full
    cfg["num_hidden_layers"] = args.layers
    rt = hb.Runtime("cuda", torch.bfloat16)
    model = hb.random_model(cfg, 0, rt)
    max_b = args.batch if args.no_points else max(args.batch, 64)
    engine = hb.Engine(model, max_tokens=max_b * args.context, max_slots=max_b, max_seq_len=args.context)
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    greedy = hb.SamplingParams(temperature=0.0)
    sampler = ClockSampler()
    sampler.start()
    windows = []

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def prefill_batch(B):
        slots = [engine.alloc_slot() for _ in range(B)]
        for s in slots:                      # one prompt per step keeps the workspace at prefill size
            engine.step([(s, rng.integers(0, V, args.prompt_len).tolist())], None)
        return slots

    def decode_device(B, steps, warmup):
        """K decode steps timed on the device: step buffer upload, graph replay, argmax."""
        slots = prefill_batch(B)
        toks = rng.integers(0, V, (steps + warmup, B)).tolist()
        out = torch.empty(B, dtype=torch.int32, device="cuda")
        def one(i):
            batch = engine._prepare([(s, [toks[i][j]]) for j, s in enumerate(slots)], "last")
            logits = engine._forward(batch)
            engine._finish(batch)
            device_choose(logits, greedy, batch.uniforms, out)
        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        lens = [engine.length(s) for s in slots]
        e0, e1 = events()
        t0 = time.time()
        e0.record()
        for i in range(warmup, warmup + steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
        windows.append((t0, time.time()))
        ms = e0.elapsed_time(e1)
        ops.check_kernel_errors()
        for s in slots:
            engine.free_slot(s)
        mean_len = sum(lens) / B + (steps + 1) / 2.0
        return ms / steps, mean_len

    def decode_e2e(B, steps, warmup):
        """The same through the public call: host token ids in, host token ids out, every step."""
        slots = prefill_batch(B)
        last = rng.integers(0, V, B).tolist()
        for _ in range(warmup):
            last = engine.step_and_choose([(s, [t]) for s, t in zip(slots, last)], greedy)
        torch.cuda.synchronize()
        t0 = time.time()
        for _ in range(steps):
            last = engine.step_and_choose([(s, [t]) for s, t in zip(slots, last)], greedy)
        dt = time.time() - t0
        windows.append((t0, t0 + dt))
        h2d, d2h = engine.h2d_bytes_last, engine.d2h_bytes_last
        for s in slots:
            engine.free_slot(s)
        return dt / steps, h2d, d2h

    result = {}
    # ---- prefill of one prompt -------------------------------------------------------------------
    if not args.no_prefill:
        T = args.prompt_len
        times = []
        for i in range(3 + 3):
            s = engine.alloc_slot()
            ids = rng.integers(0, V, T).tolist()
            e0, e1 = events()
            t0 = time.time()
            e0.record()
            engine.step([(s, ids)], "last")          # host packing, upload, every kernel, logits of the last token
            e1.record()
            torch.cuda.synchronize()
            engine.free_slot(s)
            if i >= 3:
                times.append(e0.elapsed_time(e1))
                windows.append((t0, time.time()))
        ms = statistics.median(times)
        c = model.config
        per_layer = 2 * T * (c.hidden_size * (c.q_dim + 2 * c.kv_dim) + c.q_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
        attn = 4 * c.num_attention_heads * c.head_dim * T * (T + 1) // 2
        flops = args.layers * (per_layer + attn) + 2 * c.hidden_size * c.vocab_size
        result["prefill"] = {"value": round(T / (ms / 1e3), 1), "tokens": T, "ms": round(ms, 3),
                             "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- the headline: decode at --batch -----------------------------------------------------------
    B = args.batch
    launches0 = ops.launch_count()
    ms_step, mean_len = decode_device(B, args.steps, args.warmup)
    kernels_per_step = engine.kernels_per_graph.get(B, 0) + 1       # + the argmax launch
    value = B / (ms_step / 1e3)
    step_bytes = model.weight_bytes(rows=B) + int(B * mean_len * engine.cache.bytes_per_token())
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    result["roofline"] = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                          "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]}
    if not args.no_e2e:
        s_step, h2d, d2h = decode_e2e(B, max(64, args.steps), max(8, args.warmup))
        result["e2e"] = {"value": round(B / s_step, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    if not args.no_points:
        pts = {}
        for b in (1, 64):
            ms_b, _ = decode_device(b, max(8, args.steps // 2), args.warmup)
            pts[f"decode_b{b}"] = round(b / (ms_b / 1e3), 1)
        result["points"] = pts
    if not args.no_fp32_check:
        result["fp32_check"] = fp32_check(cfg, engine)
    if not args.no_workloads and args.size == "8b" and args.layers == layers_full:
        del engine, model
        torch.cuda.empty_cache()
        for name in ("0.6b", "32b"):
            out = run_workload(name, windows)
            result.setdefault("points", {})[f"qwen3_{name}_workload_decode"] = out["decode_tok_s"]
            result.setdefault("workloads", {})[name] = out
    sampler.stop()
    clocks = sampler.summary(windows)

    line = {
        "metric": "Qwen3-8B decode tok/s at batch 1, 8, 64; prefill tok/s at 2,048 tokens",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random-init weights N(0, 0.02)",
        "impl": "ours", "gpu_launches": kernels_per_step * args.steps,
        "config": {"model": f"Qwen3-{args.size.upper()} layer sizes", "layers": args.layers, "layers_full": layers_full,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": B, "seq_len": args.prompt_len, "context": args.context, "parallelism": "single-gpu",
                   "page_size": rt.page_size, "l2": "inputs larger than L2 (all weights read every step)",
                   "cache_fill": "prefill of random prompts", "kernels_per_step": kernels_per_step,
                   "timing": "value: CUDA events around upload + graph replay + argmax; e2e: host clock, tokens in and out"},
        "clocks": clocks,
    }
    line.update(result)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
