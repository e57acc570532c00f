"""Decode and prefill throughput of the Llama4 Scout-sized model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch 8] [--context 4096]
    python bench.py --workload maverick4 | long131k      (two further workloads, a JSON line of their own)

    python bench.py --workload cpu_baseline [--reference-root DIR]      (no GPU needed)

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  `value` is decoded tokens per
second, timed on the device with CUDA events around exactly K engine steps (host token ids in, arg-max
on the device); `e2e` is the same through the Python entry point (`Model.generate`), with every
step's token ids copied from pinned host memory and the sampled ids read back; `points` and `points_e2e`
give both at batch 1 and 64.  Between timed iterations nothing is flushed: one decode step reads tens of
GB of weights, far more than the L2 holds.  `roofline` divides the bytes the timed steps had to read by
their time: every weight a step uses once -- with the experts that THOSE steps touched, counted by running
the same prompts and token feed once more, untimed, with the routing recorded -- and the cache of the live
requests.  `prefill` is one prompt of 2,048 tokens, `prefill_b8` eight of them in one call; `frac` divides
the step's flops by its time and the burst bf16 peak (`frac_of_sustained`: by the rate the library product holds
in a seconds-long loop under the power cap, which is what a step of tens of milliseconds runs at; the clocks
sampled here say the same: ~1.5 of 1.97 GHz), `frac_per_kernel` divides the time the step would
take with every kernel at its own bound (contractions at the tensor peak, but the routed experts at the
larger of that and the time to read their weights once per piece) by the measured time.
For N > 1 GPUs it prints one line that says the library is single-GPU and exits with 2.
`phases` holds device milliseconds per phase of one prefill of 2,048 tokens and of one decode step, taken
after everything else with the steps run eagerly on one stream (so their sum exceeds the step times above).

`--workload contexts`: 12 Scout layers, decode at (batch, context) of (1, 32768), (8, 32768), (64, 8192), (1, 131072)
and (8, 131072), and one prefill of 32,768 tokens, each with its roofline fraction.
`--workload cpu_baseline` times, on the host's cores, the reference's own unmodified CPU engine (compiled from
DIR with tests/golden/ref_harness.cpp, token by token as its generate loop runs it,
src/engine/llama4_cpu_engine.cpp:516-566) and this repository's plain implementation at the two tiny
configurations that lie inside what that engine computes.
`--workload maverick4`: 4 layers with Llama4 Maverick's sizes (dense and 128-expert layers alternate), 32
prompts of 64 to 2,048 tokens, 128 new tokens each.  `--workload long131k`: 12 Scout layers, one prompt of
131,072 tokens (prefilled in pieces), 256 new tokens.  Both run through `Model.generate` and are timed with
its wall-clock phases, second of two runs.
`--workload veredra`: the Veredra design (gated linear attention, windowed attention with a sink, a selective
state-space layer; gelu-gated feed-forwards; two residual streams) at two layer sizes, six layers each, beside the
dense Llama4-style decoder at the same sizes: one prefill of 2,048 tokens and decode at batch 8, device-timed, then
the time of every phase and each phase's fraction of its roofline for both models.
`--workload savenex`: the Savenex design (windowed attention with kept first tokens beside a gated delta rule in every
layer, dense and routed feed-forwards, a looped range) at two layer sizes beside Veredra's attention and
gated-linear-attention layers at the same sizes, measured the same way.
`--workload nogapel`: the Nogapel design (windowed attention with short convolutions and value mixing alternating with
attention over a cached latent; norm once, mixer and squared-relu feed-forward side by side; a gated per-token input
after every layer) at two layer sizes beside Veredra's windowed-attention layers at the same sizes, measured the
same way.
`--workload kikerax`: the Kikerax design (differential attention under a chunk mask alternating with a pair of
soft-capped attention over its own keys and a gated linear recurrent unit; norms on the sublayers' outputs; gelu
feed-forwards and experts chosen from the best groups) at two layer sizes beside Savenex's layers (attention beside a
gated delta rule, dense and routed feed-forwards) at the same sizes, measured the same way.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of Llama4 Scout (24 of its 48 layers fit one B200 in bfloat16 beside the cache).
SCOUT = {
    "architectures": ["Llama4ForCausalLM"],
    "num_hidden_layers": 24, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 8192, "intermediate_size_mlp": 16384,
    "num_local_experts": 16, "num_experts_per_tok": 1, "interleave_moe_layer_step": 1,
    "vocab_size": 202048, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "nope_layer_interval": 4, "attention_chunk_size": 8192, "use_qk_norm": True,
    "attn_temperature_tuning": True, "floor_scale": 8192, "attn_scale": 0.1,
    "tie_word_embeddings": False, "max_position_embeddings": 131072, "initializer_range": 0.02,
}
FULL_LAYERS = 48
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)) or None, "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(int(float(s[0])))
                mx = int(float(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def layer_weight_bytes(c, touched_experts: float) -> float:
    H, Q, KV = c["hidden_size"], c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    I, E = c["intermediate_size"], c["num_local_experts"]
    attn = (Q + 2 * KV) * H + H * Q
    shared = 3 * I * H
    expert = 3 * I * H
    router = E * H
    return 2.0 * (attn + shared + router + touched_experts * expert + 2 * H)


def decode_step_bytes(c, layers, batch, context, touched_experts) -> float:
    """Bytes one decode step has to read: every weight it uses once and the cache of the live requests (a layer
    with chunked attention reads the keys of the newest position's chunk only)."""
    H, V = c["hidden_size"], c["vocab_size"]
    kv_per_token = 2 * c["num_key_value_heads"] * c["head_dim"] * 2
    C, every = c["attention_chunk_size"], c["nope_layer_interval"]
    keys = 0.0
    for i in range(layers):
        nope = every > 0 and (i + 1) % every == 0
        keys += context if (nope or C <= 0) else (context - 1) % C + 1
    return (layers * layer_weight_bytes(c, touched_experts) + 2.0 * V * H + 2.0 * batch * H
            + batch * keys * kv_per_token)


def prefill_flops(c, layers, n_tokens) -> float:
    H, Q, KV = c["hidden_size"], c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    I, V, K = c["intermediate_size"], c["vocab_size"], c["num_experts_per_tok"]
    per_token = 2.0 * ((Q + 2 * KV) * H + H * Q + 3 * I * H * (1 + K) + c["num_local_experts"] * H)
    attn = 0.0
    for i in range(layers):
        nope = (i + 1) % c["nope_layer_interval"] == 0
        C = c["attention_chunk_size"]
        keys = n_tokens * (n_tokens + 1) / 2 if (nope or C >= n_tokens) else None
        if keys is None:
            full, rem = divmod(n_tokens, C)
            keys = full * C * (C + 1) / 2 + rem * (rem + 1) / 2
        attn += 4.0 * Q * keys
    return layers * per_token * n_tokens + attn + 2.0 * V * H


def prefill_bound_ms(c, layers, n_tokens, n_seqs, pieces, pk) -> float:
    """Milliseconds a prefill of n_seqs prompts of n_tokens would take with every kernel at its own bound: the
    contractions at the tensor peak, except the routed experts, which cannot be faster than reading every
    expert's weights once per piece of the step; the head reads its matrix once."""
    H, Q, KV = c["hidden_size"], c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    I, V, K, E = c["intermediate_size"], c["vocab_size"], c["num_experts_per_tok"], c["num_local_experts"]
    T = n_tokens * n_seqs
    peak, hbm = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    dense = 2.0 * T * ((Q + 2 * KV) * H + H * Q + 3 * I * H + E * H)
    routed_flops = 2.0 * T * K * 3 * I * H
    routed_bytes = 2.0 * min(E, T * K) * 3 * I * H * pieces
    attn = (prefill_flops(c, 1, n_tokens) - 2.0 * V * H - prefill_flops_linear(c, n_tokens)) * n_seqs
    per_layer = (dense + attn) / peak + max(routed_flops / peak, routed_bytes / hbm)
    return 1e3 * (layers * per_layer + 2.0 * V * H / hbm)


def prefill_flops_linear(c, n_tokens) -> float:
    H, Q, KV = c["hidden_size"], c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    I, K = c["intermediate_size"], c["num_experts_per_tok"]
    return 2.0 * ((Q + 2 * KV) * H + H * Q + 3 * I * H * (1 + K) + c["num_local_experts"] * H) * n_tokens


def run(args) -> dict:
    import torch
    from cpi_b200.api import Model
    from cpi_b200.csrc import lib as K
    from cpi_b200.engine import StepEntry

    pk = peaks()
    cfg = dict(SCOUT)
    cfg["num_hidden_layers"] = args.layers
    B, ctx, steps, warm = args.batch, args.context, args.steps, args.warmup
    max_b = max(B, 1 if args.skip_points else 64)
    t0 = time.time()
    model = Model.random(cfg, seed=0, dtype="bfloat16", max_batch=max_b, max_context=ctx, device="cuda:0")
    eng = model.engine
    torch.cuda.synchronize()
    build_s = time.time() - t0
    V = cfg["vocab_size"]
    g = torch.Generator().manual_seed(1234)

    def toks(n):
        return torch.randint(0, V, (n,), generator=g).tolist()

    out_tok = torch.empty(max_b, dtype=torch.int32, device="cuda:0")

    def timed_decode(batch, n_steps, n_warm, count_experts=True):
        """Prefill `batch` prompts so that the timed steps end at the full context; device-timed.  Returns
        (milliseconds, kernels launched, bytes the timed steps had to read, experts touched per layer and step
        as (mean, least, most))."""
        plen = ctx - (n_steps + n_warm) - 1
        prompts = [toks(plen) for _ in range(batch)]
        feed = [toks(batch) for _ in range(n_steps + n_warm)]

        def start():
            slots = [eng.acquire_slot() for _ in range(batch)]
            eng.step([StepEntry(s, p, []) for s, p in zip(slots, prompts)])
            return slots

        def one(slots, i):
            lg = eng.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            K.argmax(lg, out_tok[:batch])

        slots = start()
        for i in range(n_warm):
            one(slots, i)
        torch.cuda.synchronize()
        l0 = K.kernel_launches() + eng.graph_kernel_launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_warm, n_warm + n_steps):
            one(slots, i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = K.kernel_launches() + eng.graph_kernel_launches - l0
        for s in slots:
            eng.release_slot(s)
        # the same prompts and the same feed once more, untimed, with the routing recorded: the experts that
        # each of the timed steps touched in each layer
        per_step = []
        if count_experts:
            cap = eng.capture_routing(True)
            slots = start()
            for i in range(n_warm + n_steps):
                for lst in cap.values():
                    lst.clear()
                one(slots, i)
                if i >= n_warm:
                    torch.cuda.synchronize()
                    per_step.append([len(set(lst[0].flatten().tolist())) for lst in cap.values() if lst])
            eng.capture_routing(False)
            for s in slots:
                eng.release_slot(s)
        else:
            per_step = [[min(batch * cfg["num_experts_per_tok"], cfg["num_local_experts"])] * args.layers] * n_steps
        means = [sum(x) / len(x) for x in per_step]
        total_bytes = sum(decode_step_bytes(cfg, args.layers, batch, plen + n_warm + k + 1, m)
                          for k, m in enumerate(means))
        touched = (sum(means) / len(means), min(min(x) for x in per_step), max(max(x) for x in per_step))
        return ms, launches, total_bytes, touched

    def e2e_decode(batch, n_steps, n_warm):
        """The same through `Model.generate`: host token ids in, sampled ids read back every step."""
        plen = ctx - (n_steps + n_warm) - 1
        prompts = [toks(plen) for _ in range(batch)]
        # warm-up: the same batch for `n_warm` steps (it also captures this batch size's decode graph)
        model.generate(prompts, max_new=n_warm + 1, temperature=0.0, stop_ids=[])
        model.generate(prompts, max_new=n_steps + 1, temperature=0.0, stop_ids=[])
        st = model.stats()
        return batch * st.decode_steps / (st.decode_ms / 1e3)

    def timed_prefill(n_seqs, reps):
        times = []
        for r in range(reps + 1):                            # the first pass warms up
            slots = [eng.acquire_slot() for _ in range(n_seqs)]
            entries = [StepEntry(x, toks(pre_n), [pre_n - 1]) for x in slots]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step(entries)
            e1.record()
            torch.cuda.synchronize()
            if r:
                times.append(e0.elapsed_time(e1))
            for x in slots:
                eng.release_slot(x)
        return sorted(times)[len(times) // 2]

    def prefill_record(n_seqs, ms):
        pieces = -(-n_seqs * pre_n // eng.max_step_tokens)
        flops = n_seqs * (prefill_flops(cfg, args.layers, pre_n) - 2.0 * V * cfg["hidden_size"]) \
            + 2.0 * V * cfg["hidden_size"] * n_seqs
        sustained = pk.get("bf16_tflops_sustained")
        return {"value": round(n_seqs * pre_n / (ms / 1e3), 1), "tokens": n_seqs * pre_n, "ms": round(ms, 3),
                "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                # the same against the library product's rate in a seconds-long loop under the power cap: a step
                # of tens of milliseconds runs at those clocks, not at a burst's
                "frac_of_sustained": None if not sustained else round(flops / (ms / 1e3) / (sustained * 1e12), 4),
                "frac_per_kernel": round(prefill_bound_ms(cfg, args.layers, pre_n, n_seqs, pieces, pk) / ms, 4),
                "peak": f"bf16_tflops (burst, {pk['source']})", "tokens_per_piece": min(n_seqs * pre_n, eng.max_step_tokens)}

    # ---- prefill of 2,048 tokens: one sequence, and eight in one call ---------------------------------------
    pre_n = 2048
    pre = timed_prefill(1, 3)
    pre8 = None if args.skip_points else timed_prefill(8, 2)

    # ---- the headline: decode at the given batch ----------------------------------------------------
    clocks = ClockSampler()
    clocks.start()
    ms, launches, step_bytes, touched = timed_decode(B, steps, warm)
    clock_rec = clocks.stop()
    value = B * steps / (ms / 1e3)
    achieved = step_bytes / (ms / 1e3) / 1e9

    # ---- end to end through the Python entry point --------------------------------------------------
    e2e_value = e2e_decode(B, steps, warm)
    h2d = eng.stager.bytes_staged
    d2h = B * 4

    points, points_e2e, points_frac = {}, {}, {}
    if not args.skip_points:
        for b in (1, 64):
            k = max(4, steps if b == 1 else steps // 2)          # batch-1 steps are short: time more of them
            w = max(3, warm) + (4 if b == 1 else 0)
            m, _, nbytes, _ = timed_decode(b, k, w, count_experts=b > 1)
            points[f"decode_b{b}"] = round(b * k / (m / 1e3), 2)
            points_frac[f"decode_b{b}"] = round(nbytes / (m / 1e3) / 1e9 / pk["hbm_gbs"], 4)
            points_e2e[f"decode_b{b}"] = round(e2e_decode(b, k, w), 2)

    # ---- where the time goes: phases of one prefill and of one decode step (eager, one stream) ---------
    timer = eng.profile_phases(True)
    for it in range(2):                                      # the first pass warms the eager paths up
        timer.reset()
        s = eng.acquire_slot()
        eng.step([StepEntry(s, toks(pre_n), [pre_n - 1])])
        eng.release_slot(s)
    pre_ph = dict(timer.collect().get("prefill", {}))
    slots = [eng.acquire_slot() for _ in range(B)]
    eng.step([StepEntry(x, toks(ctx - 8), []) for x in slots])
    eng.step([StepEntry(x, toks(1), [0]) for x in slots])
    timer.reset()
    for _ in range(4):
        eng.step([StepEntry(x, toks(1), [0]) for x in slots])
    for x in slots:
        eng.release_slot(x)
    ph = timer.collect()
    eng.profile_phases(False)
    phases = {"prefill_ms": {k: round(v, 3) for k, v in pre_ph.items()},
              "decode_ms": {k: round(v / 4, 3) for k, v in ph.get("decode", {}).items()}}

    return {
        "metric": f"decode tok/s @ batch {B} (Llama4 Scout layer sizes, bf16, random weights)",
        "value": round(value, 2), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": round(ms / steps, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random-init weights N(0, 0.02)",
        "impl": "cpi_b200",
        "config": {"model": "llama4-scout-layer-sizes", "layers": args.layers, "layers_full_model": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "experts": cfg["num_local_experts"], "top_k": cfg["num_experts_per_tok"],
                   "expert_inter": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "chunk": cfg["attention_chunk_size"], "nope_interval": cfg["nope_layer_interval"],
                   "global_batch": B, "seq_len": ctx, "decode_context_end": ctx, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (a step reads > 10 GB of weights)",
                   "experts_touched_per_layer": round(touched[0], 2)},
        "e2e": {"value": round(e2e_value, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": prefill_record(1, pre),
        "prefill_b8": None if pre8 is None else prefill_record(8, pre8),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"],
                     "experts_touched": {"mean": round(touched[0], 2), "least": touched[1], "most": touched[2],
                                         "counted": "over the timed steps, in an untimed replay of the same feed"}},
        "points": points,
        "points_e2e": points_e2e,
        "points_roofline_frac": points_frac,
        "phases": phases,
        "clocks": clock_rec,
        "build_s": round(build_s, 1),
    }


def run_workload(args) -> dict:
    """BASELINE's two further workloads through the Python entry point."""
    import random

    import torch
    from cpi_b200.api import Model
    cfg = dict(SCOUT)
    if args.workload == "maverick4":
        cfg.update(num_hidden_layers=4, interleave_moe_layer_step=2, num_local_experts=128)
        cfg["rope_scaling"] = dict(cfg["rope_scaling"], factor=8.0)
        rnd = random.Random(0)
        lens, new = [rnd.randint(64, 2048) for _ in range(32)], 128
    else:
        cfg.update(num_hidden_layers=12)
        lens, new = [131072], 256
    model = Model.random(cfg, seed=0, dtype="bfloat16", max_batch=len(lens), max_context=max(lens) + new + 64,
                         device="cuda:0")
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    clocks = ClockSampler()
    for it in range(2):
        if it == 1:
            clocks.start()
        torch.cuda.synchronize()
        t0 = time.time()
        res = model.generate(prompts, max_new=new, temperature=0.0, stop_ids=[])
        torch.cuda.synchronize()
        total = time.time() - t0
    clock_rec = clocks.stop()
    model.engine.check_device_errors()
    st = model.stats()
    n_new = sum(len(r.tokens) for r in res)
    return {"metric": f"tokens/s through Model.generate, workload {args.workload} (bf16, random weights)",
            "value": round((n_new - len(lens)) / (st.decode_ms / 1e3), 1), "unit": "decoded tok/s", "n_gpus": 1,
            "higher_is_better": True, "dtype": "bf16", "impl": "cpi_b200",
            "data": "synthetic: uniform random token ids, random-init weights N(0, 0.02)",
            "config": {"model": args.workload, "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                       "experts": cfg["num_local_experts"], "moe_layer_step": cfg["interleave_moe_layer_step"],
                       "dense_inter": cfg["intermediate_size_mlp"], "expert_inter": cfg["intermediate_size"],
                       "vocab": cfg["vocab_size"], "prompts": len(lens), "prompt_tokens": sum(lens),
                       "longest_prompt": max(lens), "new_tokens_each": new, "parallelism": "single-gpu"},
            "prefill": {"value": round(sum(lens) / (st.prefill_ms / 1e3), 1), "tokens": sum(lens),
                        "ms": round(st.prefill_ms, 2)},
            "decode": {"steps": st.decode_steps, "ms": round(st.decode_ms, 2),
                       "ms_per_step": round(st.decode_ms / max(st.decode_steps, 1), 3)},
            "total_s": round(total, 3), "device_memory_gb": round(torch.cuda.max_memory_allocated() / 1e9, 1),
            "clocks": clock_rec}


def run_contexts(args) -> dict:
    """Decode at longer contexts and a long single prefill, 12 layers of Scout's sizes: (batch, context) of
    (1, 32768), (8, 32768), (64, 8192), (1, 131072), (8, 131072), and a prefill of one 32,768-token prompt.  Every
    cache is filled by a real prefill; decode steps are device-timed as in the default run; the bytes of a step
    count every weight once (experts by the expected number touched under uniform routing) and the keys and
    values that each layer's window lets through."""
    import torch
    from cpi_b200.api import Model
    from cpi_b200.csrc import lib as K
    from cpi_b200.engine import StepEntry
    pk = peaks()
    cfg = dict(SCOUT)
    L = 12
    cfg["num_hidden_layers"] = L
    V, E = cfg["vocab_size"], cfg["num_local_experts"]
    g = torch.Generator().manual_seed(7)
    out = {"metric": "decode tok/s at longer contexts (12 layers of Llama4 Scout sizes, bf16, random weights)",
           "unit": "tok/s", "n_gpus": 1, "dtype": "bf16", "impl": "cpi_b200", "higher_is_better": True,
           "data": "synthetic: uniform random token ids, random-init weights N(0, 0.02)",
           "config": {"model": "llama4-scout-layer-sizes", "layers": L, "layers_full_model": FULL_LAYERS,
                      "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                      "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "experts": E,
                      "expert_inter": cfg["intermediate_size"], "vocab": V, "chunk": cfg["attention_chunk_size"],
                      "nope_interval": cfg["nope_layer_interval"], "parallelism": "single-gpu"},
           "points": {}, "clocks": None}
    steps, warm = 16, 4
    clocks = ClockSampler()
    clocks.start()
    for batch, ctx in ((1, 32768), (8, 32768), (64, 8192), (1, 131072), (8, 131072)):
        model = Model.random(cfg, seed=0, dtype="bfloat16", max_batch=batch, max_context=ctx + 64, device="cuda:0")
        eng = model.engine
        plen = ctx - steps - warm
        slots = [eng.acquire_slot() for _ in range(batch)]
        for s in slots:                                   # one prompt at a time: the pieces stay 8,192 tokens
            eng.step([StepEntry(s, torch.randint(0, V, (plen,), generator=g).tolist(), [])])
        tok = torch.empty(batch, dtype=torch.int32, device="cuda:0")
        feed = [torch.randint(0, V, (batch,), generator=g).tolist() for _ in range(steps + warm)]

        def one(i):
            lg = eng.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            K.argmax(lg, tok)

        for i in range(warm):
            one(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warm, warm + steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
        eng.check_device_errors()
        ms = e0.elapsed_time(e1) / steps
        touched = E * (1.0 - (1.0 - 1.0 / E) ** batch)
        nbytes = decode_step_bytes(cfg, L, batch, ctx - steps / 2, touched)
        out["points"][f"decode_b{batch}_ctx{ctx}"] = {
            "tok_s": round(batch / (ms / 1e3), 1), "ms_per_step": round(ms, 3),
            "roofline_frac": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4),
            "cache_gb_held": round(sum(g_.k.numel() * 2 * 2 for g_ in eng.cache.groups) / 1e9, 1)}
        if (batch, ctx) == (1, 32768):                    # the long single prefill, on the same model
            for s in slots:
                eng.release_slot(s)
            slots = []
            times = []
            for r in range(2):
                s = eng.acquire_slot()
                p = torch.randint(0, V, (32768,), generator=g).tolist()
                e0.record()
                eng.step([StepEntry(s, p, [32767])])
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
                eng.release_slot(s)
            pms = min(times)
            # flops of 12 layers at 32,768 tokens: the linear parts per token, attention by each layer's window
            fl = prefill_flops(cfg, L, 32768)
            out["points"]["prefill_1x32768"] = {"tok_s": round(32768 / (pms / 1e3), 1), "ms": round(pms, 2),
                                                "frac": round(fl / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                                                "peak": f"bf16_tflops (burst, {pk['source']})"}
        for s in slots:
            eng.release_slot(s)
        del model, eng
        torch.cuda.empty_cache()
    out["clocks"] = clocks.stop()
    out["value"] = out["points"]["decode_b8_ctx32768"]["tok_s"]
    return out


def run_cpu_baseline(args) -> dict:
    """Tokens per second on the host's cores at the two tiny configurations inside what the reference's engine
    computes: the reference's own CPU engine (unmodified, compiled with tests/golden/ref_harness.cpp; one
    forward_token call per token, as its generate loop does) and this repository's plain implementation (whole
    sequences, one forward per generated token as its greedy loop does, and one forward over all positions)."""
    import re
    import tempfile
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_llama4 as P
    import tiny
    golden = os.path.join(ROOT, "tests", "golden")
    ref = args.reference_root
    out = {"metric": "CPU baseline: tok/s at the tiny reference-compatible configurations (float32)", "unit": "tok/s",
           "impl": "cpu_baseline", "n_gpus": 0, "cpu_threads": os.cpu_count(), "points": {}}
    exe = None
    if ref and os.path.isdir(os.path.join(ref, "src", "engine")):
        work = tempfile.mkdtemp(prefix="cpi_cpu_baseline_")
        exe = os.path.join(work, "ref_harness")
        srcs = [os.path.join(ref, p) for p in ("src/engine/llama4_cpu_engine.cpp", "src/model/safetensors_loader.cpp",
                                               "src/platform/mmap_file.cpp")]
        cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
        r = subprocess.run(["g++", "-std=c++20", "-O2", "-mavx2", "-mfma", "-fopenmp", f"-I{ref}/include",
                            f"-I{cuda_inc}", os.path.join(golden, "ref_harness.cpp"), *srcs, "-o", exe],
                           capture_output=True, text=True)
        if r.returncode != 0:
            out["reference_cpu_engine"] = "does not compile here: " + r.stderr.strip().splitlines()[-1][:200]
            exe = None
    else:
        out["reference_cpu_engine"] = "no checkout given (--reference-root DIR)"
    for name, n_tokens in (("R", 48), ("R2", 70)):
        d = tiny.make_model_dir(name)
        c = tiny.config(name)["text_config"]
        rs = c["rope_scaling"]
        tokens = tiny.random_tokens(n_tokens, c["vocab_size"], 77)
        point = {"tokens": n_tokens, "layers": c["num_hidden_layers"], "hidden": c["hidden_size"]}
        if exe:
            argv = [exe, d, os.path.join(os.path.dirname(exe), f"logits_{name}.f32"), c["vocab_size"],
                    c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                    c["num_hidden_layers"], c["num_local_experts"], c["intermediate_size"], c["intermediate_size"],
                    rs["original_max_position_embeddings"], c["rope_theta"], rs["factor"], rs["low_freq_factor"],
                    rs["high_freq_factor"], *tokens]
            best = None
            for _ in range(3):
                r = subprocess.run([str(a) for a in argv], capture_output=True, text=True, check=True)
                ms = float(re.search(r"forward_ms=([0-9.]+)", r.stderr).group(1))
                best = ms if best is None else min(best, ms)
            point["reference_cpu_engine_tok_s"] = round(n_tokens / (best / 1e3), 1)
        pc, W = P.read_config(d), P.read_weights(d)
        P.forward(pc, W, tokens)
        t0 = time.perf_counter()
        P.forward(pc, W, tokens)
        point["plain_all_positions_tok_s"] = round(n_tokens / (time.perf_counter() - t0), 1)
        t0 = time.perf_counter()
        P.greedy_generate(pc, W, tokens[:n_tokens - 8], 8)
        point["plain_greedy_tok_s"] = round(8 / (time.perf_counter() - t0), 2)
        try:
            import torch
            gpu = torch.cuda.is_available()
        except ImportError:
            gpu = False
        if gpu:                                     # the same model through this library, for scale
            from cpi_b200.api import Model
            for dtype in ("float32", "bfloat16"):
                m = Model.load(d, dtype=dtype, max_batch=1, max_context=256)
                m.generate([tokens[:n_tokens - 8]], max_new=64, temperature=0.0, stop_ids=[])
                m.generate([tokens[:n_tokens - 8]], max_new=64, temperature=0.0, stop_ids=[])
                st = m.stats()
                point[f"cpi_b200_{dtype}_decode_tok_s"] = round(st.decode_steps / (st.decode_ms / 1e3), 1)
        out["points"][name] = point
    return out


VEREDRA_SIZES = {
    # width, ff, attention (heads, kv heads, head size, window), gla (heads, key size, value size), mamba2 (heads,
    # head size, state, groups): two points with the layer shapes of 1-3 B and 7-8 B parameter models
    "w2048": dict(width=2048, ff=8192, attn=(16, 4, 128, 1024), gla=(8, 128, 256), mamba=(64, 64, 128, 8)),
    "w4096": dict(width=4096, ff=14336, attn=(32, 8, 128, 2048), gla=(16, 128, 256), mamba=(128, 64, 128, 8)),
}


def veredra_config(sz: dict, vocab: int, reps: int) -> dict:
    H, G, D, win = sz["attn"]
    gh, gk, gv = sz["gla"]
    mh, mv, mn, mg = sz["mamba"]
    mlp = {"kind": "dense", "ff": sz["ff"]}
    one = [{"type": "gla", "mixer": {"heads": gh, "dim": gk, "vdim": gv, "tau": 16.0}, "mlp": mlp},
           {"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5,
                                           "rot": {"base": 1e6, "dims": D // 2}, "mask": {"size": win}}, "mlp": mlp},
           {"type": "mamba2", "mixer": {"heads": mh, "vdim": mv, "state": mn, "groups": mg, "conv": 4,
                                        "norm_groups": mg}, "mlp": mlp}]
    return {"architecture": "Veredra", "layers": one * reps, "norm": {"eps": 1e-6}, "streams": 2, "vocab": vocab,
            "width": sz["width"], "logit_scale": 1.0, "logit_softcap": 30.0}


def llama_dense_config(sz: dict, vocab: int, layers: int) -> dict:
    """The closest model the library already had, at equal sizes: every layer attention (rotary, chunked by the
    same span as Veredra's window) and a dense SwiGLU feed-forward."""
    H, G, D, win = sz["attn"]
    cfg = dict(SCOUT)
    cfg.update({"num_hidden_layers": layers, "hidden_size": sz["width"], "num_attention_heads": H,
                "num_key_value_heads": G, "head_dim": D, "intermediate_size": sz["ff"], "intermediate_size_mlp": sz["ff"],
                "interleave_moe_layer_step": 1 << 20, "vocab_size": vocab, "nope_layer_interval": 0,
                "attention_chunk_size": win, "attn_temperature_tuning": False})
    cfg.pop("moe_layers", None)
    return cfg


def measure_config(cfg, vocab, T, B, toks):
    """One model drawn from `cfg`: a prompt of T tokens (median of five after a warm-up), decode at batch B on a
    context of T - 64 (32 steps, device-timed), then the phases of one prompt and of four decode steps (eager, one
    stream)."""
    import torch
    from cpi_b200.engine import Engine, StepEntry
    eng = Engine.from_random(cfg, 0, dtype="bfloat16", max_tokens=(B + 1) * (T + 128), max_seqs=B + 1,
                             max_seq_len=T + 128)
    res = {}

    def prefill():
        s = eng.acquire_slot()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([StepEntry(s, toks(T), [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        eng.release_slot(s)
        return e0.elapsed_time(e1)

    times = sorted(prefill() for _ in range(6))[:-1]          # the first (slowest) pass warms up
    res["prefill_ms"] = round(times[len(times) // 2], 3)
    res["prefill_tok_s"] = round(T / (res["prefill_ms"] / 1e3), 1)
    slots = [eng.acquire_slot() for _ in range(B)]
    eng.step([StepEntry(s, toks(T - 64), []) for s in slots])
    for _ in range(8):
        eng.step([StepEntry(s, toks(1), [0]) for s in slots])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(32):
        eng.step([StepEntry(s, toks(1), [0]) for s in slots])
    e1.record()
    torch.cuda.synchronize()
    res["decode_ms_per_step"] = round(e0.elapsed_time(e1) / 32, 4)
    res["decode_tok_s"] = round(B / (res["decode_ms_per_step"] / 1e3), 1)
    res["graphs"] = bool(eng.use_graphs)
    timer = eng.profile_phases(True)
    for _ in range(4):
        eng.step([StepEntry(s, toks(1), [0]) for s in slots])
    for s in slots:
        eng.release_slot(s)
    s = eng.acquire_slot()
    eng.step([StepEntry(s, toks(T), [T - 1])])
    eng.release_slot(s)
    ph = timer.collect()
    eng.profile_phases(False)
    res["phases_ms"] = {"prefill": {k: round(v, 4) for k, v in ph.get("prefill", {}).items()},
                        "decode_per_step": {k: round(v / 4, 4) for k, v in ph.get("decode", {}).items()}}
    del eng
    torch.cuda.empty_cache()
    return res



def run_veredra(args) -> dict:
    """Prefill and decode of Veredra at two layer sizes beside the dense Llama4-style decoder at equal sizes, with
    the time of every phase per layer that has it and each phase's share of its roofline (products: flops over the
    measured bf16 rate in prefill, weight bytes over the measured copy rate in decode; attention: flops / cache
    bytes; recurrences, norms and stream mixing: bytes)."""
    import torch
    from cpi_b200.engine import Engine, StepEntry

    pk = peaks()
    vocab, reps, T, B = 32000, 2, 2048, 8
    g = torch.Generator().manual_seed(7)
    toks = lambda n: torch.randint(0, vocab, (n,), generator=g).tolist()
    out = {"metric": "tokens/s, Veredra beside the dense decoder at equal layer sizes (bf16, random weights)",
           "unit": "tokens/s", "dtype": "bf16", "data": "synthetic", "peaks": pk, "points": {}}

    measure = lambda cfg, n_layers: measure_config(cfg, vocab, T, B, toks)

    for name, sz in VEREDRA_SIZES.items():
        W, ff = sz["width"], sz["ff"]
        H, G, D, win = sz["attn"]
        gh, gk, gv = sz["gla"]
        mh, mv, mn, mg = sz["mamba"]
        n_layers = 3 * reps
        ver = measure(veredra_config(sz, vocab, reps), n_layers)
        lla = measure(llama_dense_config(sz, vocab, n_layers), n_layers)
        tf, bw = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
        keys = sum(min(t + 1, win) for t in range(T))
        # per layer that has the phase: what the phase must do at least
        attn_flops = 4.0 * D * H * keys
        attn_dec_bytes = B * min(T, win) * G * 2 * D * 2.0
        mlp_params, qkv_attn, wo_attn = 3.0 * W * ff, (H + 2 * G) * D * W, H * D * W
        gla_proj = (2 * gh * gk + 2 * gh * gv) * W + 16 * W + 16 * gh * gk
        inner = mh * mv
        mamba_proj = (2 * inner + 2 * mg * mn + mh) * W
        scan_prefill_bytes = {"gla": T * (3 * gh * gk + 2 * gh * gv) * 4.0, "mamba2": T * (2 * mg * mn + 2 * inner + mh) * 4.0}
        scan_decode_bytes = {"gla": B * gh * gk * gv * 8.0, "mamba2": B * mh * mn * mv * 8.0}

        def frac(ms, flops=0.0, nbytes=0.0):
            return None if not ms else round(max(flops / tf, nbytes / bw) / (ms / 1e3), 4)

        vp, vd = ver["phases_ms"]["prefill"], ver["phases_ms"]["decode_per_step"]
        lp, ld = lla["phases_ms"]["prefill"], lla["phases_ms"]["decode_per_step"]
        roof = {
            "mlp": {"veredra": {"prefill": frac(vp.get("mlp", 0) / n_layers, 2.0 * T * mlp_params),
                                "decode": frac(vd.get("mlp", 0) / n_layers, nbytes=2.0 * mlp_params)},
                    "dense": {"prefill": frac(lp.get("mlp", 0) / n_layers, 2.0 * T * mlp_params),
                              "decode": frac(ld.get("mlp", 0) / n_layers, nbytes=2.0 * mlp_params)}},
            "attention": {"veredra": {"prefill": frac(vp.get("attention", 0) / reps, attn_flops),
                                      "decode": frac(vd.get("attention", 0) / reps, nbytes=attn_dec_bytes)},
                          "dense": {"prefill": frac(lp.get("attention", 0) / n_layers, attn_flops),
                                    "decode": frac(ld.get("attention", 0) / n_layers, nbytes=attn_dec_bytes)}},
            "qkv_and_wo": {"veredra": {"prefill": frac((vp.get("qkv", 0) + vp.get("wo", 0)) / reps,
                                                       2.0 * T * (qkv_attn + wo_attn + gla_proj + gh * gv * W + mamba_proj + inner * W)),
                                       "decode": frac((vd.get("qkv", 0) + vd.get("wo", 0)) / reps, nbytes=2.0 * (
                                           qkv_attn + wo_attn + gla_proj + gh * gv * W + mamba_proj + inner * W))},
                           "dense": {"prefill": frac((lp.get("qkv", 0) + lp.get("wo", 0)) / n_layers, 2.0 * T * (qkv_attn + wo_attn)),
                                     "decode": frac((ld.get("qkv", 0) + ld.get("wo", 0)) / n_layers, nbytes=2.0 * (qkv_attn + wo_attn))}},
            "scan (gla + mamba2, no like kernel)": {"veredra": {
                "prefill": frac(vp.get("scan", 0) / reps, nbytes=sum(scan_prefill_bytes.values())),
                "decode": frac(vd.get("scan", 0) / reps, nbytes=sum(scan_decode_bytes.values()))}},
            "norms_and_residual": {
                # two stream kernels a layer: each reads and writes both float32 streams, reads y, writes h
                "veredra": {"prefill": frac(vp.get("rmsnorm", 0) / n_layers, nbytes=T * W * 2 * (2 * 2 * 4 + 4 + 2.0))},
                "dense": {"prefill": frac(lp.get("rmsnorm", 0) / n_layers, nbytes=T * W * 2 * (4 + 2.0))}},
        }
        out["points"][name] = {"sizes": sz, "layers": n_layers, "prefill_tokens": T, "decode_batch": B,
                               "decode_context": T - 64, "veredra": ver, "dense": lla, "fraction_of_roofline": roof}
    big = out["points"]["w4096"]
    out["value"] = big["veredra"]["decode_tok_s"]
    out["config"] = {"model": "Veredra, 6 layers (gla, attention, mamba2) x 2, two streams", "global_batch": B,
                     "seq_len": T, "parallelism": "single GPU", "l2": "weights of a step exceed the L2"}
    return out


SAVENEX_SIZES = {
    # width, dense ff, experts (count, top, ff each, shared ff), left = attention (heads, kv heads, head size, window,
    # kept first tokens), right = gated delta rule (heads, q/k heads, key size, value size, taps): two points with
    # the layer shapes of 1-3 B and 7-8 B parameter models
    "w2048": dict(width=2048, ff=8192, moe=(16, 2, 2048, 2048), left=(16, 4, 128, 1024, 64), right=(8, 4, 128, 256, 4)),
    "w4096": dict(width=4096, ff=14336, moe=(16, 2, 3584, 3584), left=(32, 8, 128, 2048, 64), right=(16, 8, 128, 256, 4)),
}


def savenex_config(sz: dict, vocab: int) -> dict:
    """Four layers (dense, routed, dense, routed feed-forwards); the two in the middle run twice: six layer runs."""
    H, G, D, win, keep = sz["left"]
    rh, rg, rk, rv, taps = sz["right"]
    E, top, eff, sff = sz["moe"]
    mixer = {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5,
                      "rot": {"base": 1e6, "dims": D, "scaling": {"factor": 2.0}},
                      "mask": {"size": win, "keep_first": keep}},
             "right": {"heads": rh, "kv_heads": rg, "dim": rk, "vdim": rv, "conv": taps}}
    dense = {"kind": "dense", "ff": sz["ff"], "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top}, "shared": {"ff": sff}}
    return {"architecture": "Savenex", "layers": [{"type": "parallel", "mixer": mixer, "mlp": m} for m in (dense, moe, dense, moe)],
            "loop": {"start": 1, "stop": 3, "times": 2}, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "vocab": vocab,
            "width": sz["width"]}


def veredra_pairs_config(sz: dict, vocab: int, pairs: int) -> dict:
    """The closest model the library had: Veredra with as many (windowed attention, gated linear attention) pairs of
    layers as Savenex has layer runs, at the same head counts, head sizes, window and feed-forward size; one residual."""
    H, G, D, win, _ = sz["left"]
    rh, _, rk, rv, _ = sz["right"]
    mlp = {"kind": "dense", "ff": sz["ff"]}
    pair = [{"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5,
                                            "rot": {"base": 1e6, "dims": D // 2}, "mask": {"size": win}}, "mlp": mlp},
            {"type": "gla", "mixer": {"heads": rh, "dim": rk, "vdim": rv, "tau": 16.0}, "mlp": None}]
    return {"architecture": "Veredra", "layers": pair * pairs, "norm": {"eps": 1e-6}, "vocab": vocab,
            "width": sz["width"], "logit_scale": 1.0, "logit_softcap": 30.0}


def run_savenex(args) -> dict:
    """Prefill and decode of Savenex at two layer sizes beside Veredra (attention and gated-linear-attention layers in
    pairs) at equal sizes, with the time of every phase per layer run that has it and each phase's share of its
    roofline: products by flops over the measured bf16 rate in prefill and by weight bytes over the measured copy
    rate in decode; attention by flops / cache bytes; recurrences and row kernels by bytes."""
    import torch

    pk = peaks()
    vocab, T, B, runs = 32000, 2048, 8, 6
    g = torch.Generator().manual_seed(7)
    toks = lambda n: torch.randint(0, vocab, (n,), generator=g).tolist()
    out = {"metric": "tokens/s, Savenex beside Veredra at equal layer sizes (bf16, random weights)",
           "unit": "tokens/s", "dtype": "bf16", "data": "synthetic", "peaks": pk, "points": {}}
    tf, bw = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    for name, sz in SAVENEX_SIZES.items():
        W, ff = sz["width"], sz["ff"]
        H, G, D, win, keep = sz["left"]
        rh, rg, rk, rv, taps = sz["right"]
        E, top, eff, sff = sz["moe"]
        sav = measure_config(savenex_config(sz, vocab), vocab, T, B, toks)
        ver = measure_config(veredra_pairs_config(sz, vocab, runs), vocab, T, B, toks)
        sp, sd = sav["phases_ms"]["prefill"], sav["phases_ms"]["decode_per_step"]
        vp, vd = ver["phases_ms"]["prefill"], ver["phases_ms"]["decode_per_step"]

        def frac(ms, flops=0.0, nbytes=0.0):
            return None if not ms else round(max(flops / tf, nbytes / bw) / (ms / 1e3), 4)

        def both(sm, s_work, vm, v_work, per_s=runs, per_v=runs):
            """{model: {prefill, decode}} for a phase (or a sum of phases) that both models have."""
            get = lambda ph, names: sum(ph.get(n, 0) for n in names)
            return {"savenex": {"prefill": frac(get(sp, sm) / per_s, *s_work[0]), "decode": frac(get(sd, sm) / per_s, *s_work[1])},
                    "veredra": {"prefill": frac(get(vp, vm) / per_v, *v_work[0]), "decode": frac(get(vd, vm) / per_v, *v_work[1])}}

        keys_win = sum(min(t + 1, win) for t in range(T))
        keys_kept = sum(min(keep, max(0, t + 1 - win)) for t in range(T))
        ctx = T - 64
        attn_dec = lambda k: B * k * G * 2 * D * 2.0
        s_proj = ((H + 2 * G) * D + H * D) * W + ((2 * rg * rk + rh * rv + rh + 32) * W + 16 * (rh * rk + rh * rv) + rh * rv * W)
        v_proj = ((H + 2 * G) * D + H * D) * W + ((2 * rh * rk + 2 * rh * rv + 16) * W + 16 * rh * rk + rh * rv * W)
        s_scan_p = T * (2 * rg * rk + rh * rk + 2 * rh * rv + rh) * 4.0
        v_scan_p = T * (3 * rh * rk + 2 * rh * rv) * 4.0
        state = B * rh * rk * rv * 8.0
        dense_params, moe_flops = 3.0 * W * ff, 2.0 * T * 3.0 * W * (top * eff + sff)
        touched = min(E, B * top) * 0.8                      # experts a decode step of B tokens reads, roughly
        roof = {
            "attention (window + kept first tokens / window + sink; tensor-core kernels)": both(
                ["attention"], ((4.0 * D * H * (keys_win + keys_kept),), (0.0, attn_dec(min(ctx, win) + min(keep, max(0, ctx - win))))),
                ["attention"], ((4.0 * D * H * keys_win,), (0.0, attn_dec(min(ctx, win))))),
            "recurrence (gated delta rule / gated linear attention; linear_scan)": both(
                ["scan"], ((0.0, s_scan_p), (0.0, state)), ["scan"], ((0.0, v_scan_p), (0.0, state))),
            "mixer projections in and out": both(["qkv", "wo"], ((2.0 * T * s_proj,), (0.0, 2.0 * s_proj)),
                                                 ["qkv", "wo"], ((2.0 * T * v_proj,), (0.0, 2.0 * v_proj))),
            "row kernels of the mixers (rotation and cache write, convolution, unit vectors, gated norm, branch sum / the same without convolution and sum)": both(
                ["kv_store", "conv", "gated_norm", "combine"],
                ((0.0, T * 4.0 * ((H + 2 * G) * D * 1.5 + 4 * (2 * rg * rk + rh * rv) + 3.5 * rh * rv + 3 * W)),) * 2,
                ["kv_store", "gated_norm"], ((0.0, T * 4.0 * ((H + 2 * G) * D * 1.5 + 3.5 * rh * rv)),) * 2),
            "dense feed-forward and the shared expert (clamped and silu gates / gelu gate)": both(
                ["mlp"], ((2.0 * T * (dense_params + 3.0 * W * sff),), (0.0, 2.0 * (dense_params + 3.0 * W * sff))),
                ["mlp"], ((2.0 * T * dense_params,), (0.0, 2.0 * dense_params)), per_s=runs / 2),
            "routed experts (no like kernel in Veredra; Llama4's run the same grouped products)": {
                "savenex": {"prefill": frac(sum(sp.get(n, 0) for n in ("moe_router", "moe_expert", "moe_merge")) / (runs / 2),
                                            2.0 * T * 3.0 * W * top * eff),
                            "decode": frac(sum(sd.get(n, 0) for n in ("moe_router", "moe_expert", "moe_merge")) / (runs / 2),
                                           nbytes=2.0 * touched * 3.0 * W * eff)}},
            "norms and the residual": both(["rmsnorm"], ((0.0, T * W * 2 * (4 + 4 + 4 + 2.0)),) * 2,
                                           ["rmsnorm"], ((0.0, T * W * (4 + 2.0)),) * 2, per_s=runs, per_v=1.5 * runs),
        }
        out["points"][name] = {"sizes": sz, "layer_runs": runs, "prefill_tokens": T, "decode_batch": B, "decode_context": ctx,
                               "savenex": sav, "veredra": ver, "fraction_of_roofline": roof}
    big = out["points"]["w4096"]
    out["value"] = big["savenex"]["decode_tok_s"]
    out["config"] = {"model": "Savenex, 4 layers (attention beside a gated delta rule; dense and routed feed-forwards), "
                              "layers 1-2 run twice", "global_batch": B, "seq_len": T, "parallelism": "single GPU",
                     "l2": "weights of a step exceed the L2"}
    return out


NOGAPEL_SIZES = {
    # width, ff, windowed attention (heads, kv heads, head size, window, taps), latent attention (heads, plain and
    # rotated key size, value size, query rank, latent rank), elements of the per-token input: two points with the
    # layer shapes of 1-3 B and 7-8 B parameter models
    "w2048": dict(width=2048, ff=8192, attn=(16, 4, 128, 1024, 4), latent=(16, 128, 64, 128, 768, 512), side=64),
    "w4096": dict(width=4096, ff=14336, attn=(32, 8, 128, 2048, 4), latent=(32, 128, 64, 128, 1536, 512), side=128),
}


def nogapel_config(sz: dict, vocab: int, pairs: int) -> dict:
    """(windowed attention, latent attention) x pairs, every layer with a feed-forward and the per-token input."""
    H, G, D, win, taps = sz["attn"]
    lh, ld, lr, lv, qr, kr = sz["latent"]
    mlp = {"kind": "dense", "ff": sz["ff"]}
    pair = [{"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "conv": taps,
                                            "v_mix": True, "mask": {"size": win},
                                            "rot": {"base": 1e6, "dims": D, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0,
                                                                                        "original": 8192}}}, "mlp": mlp},
            {"type": "latent_attention", "mixer": {"heads": lh, "dim": ld, "rot_dim": lr, "vdim": lv, "q_rank": qr,
                                                   "kv_rank": kr, "scale": (ld + lr) ** -0.5,
                                                   "rot": {"base": 1e4, "dims": lr}}, "mlp": mlp}]
    return {"architecture": "Nogapel", "layers": pair * pairs, "norm": {"eps": 1e-6}, "token_side": {"dim": sz["side"]},
            "vocab": vocab, "width": sz["width"]}


def veredra_attention_config(sz: dict, vocab: int, layers: int) -> dict:
    """The closest model the library had: Veredra with windowed-attention layers only (a sink, a rotation of half of
    each head) and gelu-gated feed-forwards, at the same head counts, head size, window, width and feed-forward size."""
    H, G, D, win, _ = sz["attn"]
    one = {"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5,
                                          "rot": {"base": 1e6, "dims": D // 2}, "mask": {"size": win}},
           "mlp": {"kind": "dense", "ff": sz["ff"]}}
    return {"architecture": "Veredra", "layers": [one] * layers, "norm": {"eps": 1e-6}, "vocab": vocab,
            "width": sz["width"], "logit_scale": 1.0, "logit_softcap": 30.0}


def run_nogapel(args) -> dict:
    """Prefill and decode of Nogapel at two layer sizes beside Veredra's windowed-attention layers at equal sizes, with
    the time of every phase per layer that has it and each phase's share of its roofline: products by flops over the
    measured bf16 rate in prefill and by weight bytes over the measured copy rate in decode; attention by flops / cache
    bytes; row kernels by bytes."""
    import torch

    pk = peaks()
    vocab, T, B, pairs = 32000, 2048, 8, 3
    n_layers = 2 * pairs
    g = torch.Generator().manual_seed(7)
    toks = lambda n: torch.randint(0, vocab, (n,), generator=g).tolist()
    out = {"metric": "tokens/s, Nogapel beside Veredra's attention layers at equal layer sizes (bf16, random weights)",
           "unit": "tokens/s", "dtype": "bf16", "data": "synthetic", "peaks": pk, "points": {}}
    tf, bw = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    sizes = {k: v for k, v in NOGAPEL_SIZES.items() if not args.sizes or k in args.sizes.split(",")}
    for name, sz in sizes.items():
        W, ff = sz["width"], sz["ff"]
        H, G, D, win, taps = sz["attn"]
        lh, ld, lr, lv, qr, kr = sz["latent"]
        nog = measure_config(nogapel_config(sz, vocab, pairs), vocab, T, B, toks)
        ver = measure_config(veredra_attention_config(sz, vocab, n_layers), vocab, T, B, toks)
        np_, nd = nog["phases_ms"]["prefill"], nog["phases_ms"]["decode_per_step"]
        vp, vd = ver["phases_ms"]["prefill"], ver["phases_ms"]["decode_per_step"]

        def frac(ms, flops=0.0, nbytes=0.0):
            return None if not ms else round(max(flops / tf, nbytes / bw) / (ms / 1e3), 4)

        def both(nm, n_work, vm, v_work, per_n, per_v=n_layers):
            get = lambda ph, names: sum(ph.get(n, 0) for n in names)
            res = {"nogapel": {"prefill": frac(get(np_, nm) / per_n, *n_work[0]), "decode": frac(get(nd, nm) / per_n, *n_work[1])}}
            if vm is not None:
                res["veredra"] = {"prefill": frac(get(vp, vm) / per_v, *v_work[0]), "decode": frac(get(vd, vm) / per_v, *v_work[1])}
            return res

        ctx = T - 64
        keys_win = sum(min(t + 1, win) for t in range(T))
        keys_all = T * (T + 1) // 2
        row = kr + lr
        attn_dec = B * min(ctx, win) * G * 2 * D * 2.0
        # attention over the cached rows: scores over kr + lr elements, values over kr, all heads on the same rows
        lat_flops, lat_dec_bytes = 2.0 * lh * keys_all * (row + kr), B * ctx * row * 2.0
        a_proj = ((H + 2 * G) * D + H * D) * W
        l_proj = (qr + row) * W + qr * lh * (ld + lr) + lh * ld * kr + lh * kr * lv + lh * lv * W
        roof = {
            "windowed attention (tensor-core kernels both)": both(
                ["attention"], ((4.0 * D * H * keys_win,), (0.0, attn_dec)), ["attention"], ((4.0 * D * H * keys_win,), (0.0, attn_dec)),
                per_n=pairs),
            "attention over the cached latent (like kernel: the windowed attention above)": both(
                ["latent_attention"], ((lat_flops,), (max(0.0, 2.0 * B * lh * ctx * (row + kr)), lat_dec_bytes)), None, None, per_n=pairs),
            "mixer projections in and out": both(["qkv", "wo"], ((2.0 * T * (a_proj + l_proj),), (0.0, 2.0 * (a_proj + l_proj))),
                                                 ["qkv", "wo"], ((2.0 * T * a_proj,), (0.0, 2.0 * a_proj)), per_n=pairs),
            "feed-forward products (squared relu / gelu gate in the epilogue)": both(
                ["mlp"], ((2.0 * T * 2.0 * W * ff,), (0.0, 2.0 * 2.0 * W * ff)),
                ["mlp"], ((2.0 * T * 3.0 * W * ff,), (0.0, 2.0 * 3.0 * W * ff)), per_n=n_layers),
            "row kernels of the mixers (convolution, head norm, rotation, value mixing, cache write / rotation and cache write)": both(
                ["kv_store", "conv"], ((0.0, T * ((H + 2 * G) * D * (4 * 3 + 2.0) + (qr + row) * 4.0 + lh * (ld + lr) * 4.0 + lh * row * 2.0) / 2),) * 2,
                ["kv_store"], ((0.0, T * (H + 2 * G) * D * (4 + 2.0)),) * 2, per_n=n_layers),
            "norms and the residual (rmsnorm)": both(["rmsnorm"], ((0.0, T * (W * (4 + 2.0) + qr * (4 + 2.0) / 2)),) * 2,
                                                     ["rmsnorm"], ((0.0, T * W * (4 + 2.0)),) * 2, per_n=n_layers, per_v=2 * n_layers),
            "gated per-token input (no like kernel)": both(["side_input"], ((0.0, T * W * 8.0),) * 2, None, None, per_n=n_layers),
        }
        out["points"][name] = {"sizes": sz, "layers": n_layers, "prefill_tokens": T, "decode_batch": B, "decode_context": ctx,
                               "nogapel": nog, "veredra": ver, "fraction_of_roofline": roof}
    big = out["points"][sorted(out["points"])[-1]]
    out["value"] = big["nogapel"]["decode_tok_s"]
    out["config"] = {"model": "Nogapel, (windowed attention, latent attention) x 3, per-token input after every layer",
                     "global_batch": B, "seq_len": T, "parallelism": "single GPU", "l2": "weights of a step exceed the L2"}
    return out


KIKERAX_SIZES = {
    # width, dense ff, experts (count, top, ff each, shared ff, groups, kept), attention heads (heads, kv heads, head
    # size = value size, chunk), the recurrent unit (channels, blocks, taps): two points with the layer shapes of 1-3 B
    # and 7-8 B parameter models
    "w2048": dict(width=2048, ff=8192, moe=(16, 2, 2048, 2048, 4, 2), attn=(16, 4, 128, 1024), unit=(2048, 16, 4)),
    "w4096": dict(width=4096, ff=14336, moe=(16, 2, 3584, 3584, 4, 2), attn=(32, 8, 128, 2048), unit=(4096, 16, 4)),
}


def kikerax_config(sz: dict, vocab: int, pairs: int) -> dict:
    """(differential attention + dense feed-forward, pair + routed experts) x pairs."""
    H, G, D, chunk = sz["attn"]
    C, blocks, taps = sz["unit"]
    E, top, eff, sff, groups, keep = sz["moe"]
    diff = {"type": "attention", "mlp": {"kind": "dense", "ff": sz["ff"]},
            "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "diff": 0.5, "mask": {"size": chunk},
                      "rot": {"base": 1e6, "dims": D // 2, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    pair = {"type": "parallel",
            "mlp": {"kind": "moe", "expert": {"ff": eff}, "shared": {"ff": sff},
                    "router": {"experts": E, "top": top, "scale": 2.0, "groups": {"count": groups, "keep": keep}}},
            "mixer": {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "softcap": 30.0,
                               "q_temp": {"coef": 0.1, "every": 1024}},
                      "right": {"width": C, "blocks": blocks, "conv": taps}, "left_scale": 0.7, "right_scale": 0.7}}
    return {"architecture": "Kikerax", "layers": [diff, pair] * pairs, "norm": {"eps": 1e-6}, "vocab": vocab,
            "width": sz["width"], "logit_softcap": 30.0}


def savenex_like_kikerax_config(sz: dict, vocab: int, layers: int) -> dict:
    """The closest model the library had: Savenex layers (attention beside a gated delta rule; dense and routed
    feed-forwards alternating) at the same width, head counts, head size, expert sizes; the attention sees everything,
    the delta rule's state has as many value channels as the recurrent unit has channels."""
    H, G, D, _ = sz["attn"]
    C, _, taps = sz["unit"]
    E, top, eff, sff, _, _ = sz["moe"]
    mixer = {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "rot": {"base": 1e6, "dims": D}},
             "right": {"heads": C // 256, "kv_heads": max(1, C // 512), "dim": 128, "vdim": 256, "conv": taps}}
    dense = {"kind": "dense", "ff": sz["ff"], "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top}, "shared": {"ff": sff}}
    return {"architecture": "Savenex", "layers": [{"type": "parallel", "mixer": mixer, "mlp": m} for m in (dense, moe) * (layers // 2)],
            "norm": {"eps": 1e-6}, "vocab": vocab, "width": sz["width"]}


def run_kikerax(args) -> dict:
    """Prefill and decode of Kikerax at two layer sizes beside Savenex layers at equal sizes, with the time of every
    phase per layer that has it and each phase's share of its roofline: products by flops over the measured bf16 rate in
    prefill and by weight bytes over the measured copy rate in decode; attention by flops / cache bytes; recurrences and
    row kernels by bytes."""
    import torch

    pk = peaks()
    vocab, T, B, pairs = 32000, 2048, 8, 2
    n_layers = 2 * pairs
    g = torch.Generator().manual_seed(7)
    toks = lambda n: torch.randint(0, vocab, (n,), generator=g).tolist()
    out = {"metric": "tokens/s, Kikerax beside Savenex layers at equal layer sizes (bf16, random weights)",
           "unit": "tokens/s", "dtype": "bf16", "data": "synthetic", "peaks": pk, "points": {}}
    tf, bw = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    sizes = {k: v for k, v in KIKERAX_SIZES.items() if not args.sizes or k in args.sizes.split(",")}
    for name, sz in sizes.items():
        W, ff = sz["width"], sz["ff"]
        H, G, D, chunk = sz["attn"]
        C, blocks, taps = sz["unit"]
        E, top, eff, sff, _, _ = sz["moe"]
        kik = measure_config(kikerax_config(sz, vocab, pairs), vocab, T, B, toks)
        sav = measure_config(savenex_like_kikerax_config(sz, vocab, n_layers), vocab, T, B, toks)
        kp, kd = kik["phases_ms"]["prefill"], kik["phases_ms"]["decode_per_step"]
        sp, sd = sav["phases_ms"]["prefill"], sav["phases_ms"]["decode_per_step"]

        def frac(ms, flops=0.0, nbytes=0.0):
            return None if not ms else round(max(flops / tf, nbytes / bw) / (ms / 1e3), 4)

        def both(km, k_work, sm, s_work, per_k, per_s=n_layers):
            get = lambda ph, names: sum(ph.get(n, 0) for n in names)
            res = {"kikerax": {"prefill": frac(get(kp, km) / per_k, *k_work[0]), "decode": frac(get(kd, km) / per_k, *k_work[1])}}
            if sm is not None:
                res["savenex"] = {"prefill": frac(get(sp, sm) / per_s, *s_work[0]), "decode": frac(get(sd, sm) / per_s, *s_work[1])}
            return res

        ctx = T - 64
        keys_all = T * (T + 1) // 2
        keys_chunk = sum(t % chunk + 1 for t in range(T))
        # per layer pair: two maps under the chunk mask, one map over everything
        k_attn_flops = 4.0 * D * H * (2 * keys_chunk + keys_all)
        k_attn_dec = B * G * D * 2.0 * (3 * (ctx % chunk + 1) + 2 * ctx)       # k, k2, v of the chunk; k, v of everything
        s_attn_flops, s_attn_dec = 4.0 * D * H * keys_all, B * ctx * G * 2 * D * 2.0
        n = C // blocks
        d_proj = (2 * (H + G) * D + G * D + H + H * D) * W                      # q, k of two maps, v, gates, o
        l_proj = ((H + G) * D + H + H * D) * W                                  # q, k, gates, o
        u_proj = 3 * C * W + 2 * C * n                                          # y, x, o, the two block-diagonal gates
        rh, rg = C // 256, max(1, C // 512)
        s_proj = ((H + 2 * G) * D + H * D) * W + ((2 * rg * 128 + rh * 256 + rh + 32) * W + 16 * (rh * 128 + rh * 256) + rh * 256 * W)
        dense_params = 2.0 * W * ff
        s_dense_params = 3.0 * W * ff
        touched = min(E, B * top) * 0.8
        roof = {
            "attention (two maps under a chunk mask, one soft-capped map over everything / one map over everything; tensor-core kernels)": both(
                ["attention"], ((k_attn_flops,), (0.0, k_attn_dec)), ["attention"], ((s_attn_flops,), (0.0, s_attn_dec)), per_k=pairs),
            "recurrence (gated linear recurrent unit, rglru_scan / gated delta rule, linear_scan)": both(
                ["scan"], ((0.0, T * C * (4 * 4 + 2.0)), (0.0, B * C * (4 * 6 + 2.0))),
                ["scan"], ((0.0, T * (2 * rg * 128 + rh * 128 + 2 * rh * 256 + rh) * 4.0), (0.0, B * rh * 128 * 256 * 8.0)), per_k=pairs),
            "mixer projections in and out (with the unit's gate products)": both(
                ["qkv", "wo", "gates"], ((2.0 * T * (d_proj + l_proj + u_proj),), (0.0, 2.0 * (d_proj + l_proj + u_proj))),
                ["qkv", "wo"], ((2.0 * T * s_proj,), (0.0, 2.0 * s_proj)), per_k=pairs),
            "row kernels of the mixers (norm, rotation, cache write, what follows attention per head, convolution / rotation, cache write, convolution, unit vectors, gated norm, branch sum)": both(
                ["kv_store", "head_post", "conv"],
                ((0.0, T * ((2 * (H + G) * D + G * D) * (4 + 2.0) + (H + G) * D * (4 + 2.0) + 3 * H * D * 2 * 2.0 + C * 8.0)),) * 2,
                ["kv_store", "conv", "gated_norm", "combine"],
                ((0.0, T * 4.0 * ((H + 2 * G) * D * 1.5 + 4 * (2 * rg * 128 + rh * 256) + 3.5 * rh * 256 + 3 * W)),) * 2, per_k=pairs),
            "dense feed-forward and the shared expert (gelu in the up product's epilogue, silu gate / clamped and silu gates)": both(
                ["mlp"], ((2.0 * T * (dense_params + 3.0 * W * sff),), (0.0, 2.0 * (dense_params + 3.0 * W * sff))),
                ["mlp"], ((2.0 * T * (s_dense_params + 3.0 * W * sff),), (0.0, 2.0 * (s_dense_params + 3.0 * W * sff))),
                per_k=pairs, per_s=n_layers / 2),
            "routed experts (choice from the best groups / the best logits; the same grouped products)": both(
                ["moe_router", "moe_expert", "moe_merge"], ((2.0 * T * 3.0 * W * top * eff,), (0.0, 2.0 * touched * 3.0 * W * eff)),
                ["moe_router", "moe_expert", "moe_merge"], ((2.0 * T * 3.0 * W * top * eff,), (0.0, 2.0 * touched * 3.0 * W * eff)),
                per_k=pairs, per_s=n_layers / 2),
            "norms and the residual (one kernel per sublayer: sum, norm, add, next input / hc_step with one stream)": both(
                ["rmsnorm"], ((0.0, T * W * (4 + 4 + 4 + 2.0)),) * 2, ["rmsnorm"], ((0.0, T * W * 2 * (4 + 4 + 4 + 2.0) / 2),) * 2,
                per_k=2 * n_layers, per_s=2 * n_layers),
        }
        out["points"][name] = {"sizes": sz, "layers": n_layers, "prefill_tokens": T, "decode_batch": B, "decode_context": ctx,
                               "kikerax": kik, "savenex": sav, "fraction_of_roofline": roof}
    big = out["points"][sorted(out["points"])[-1]]
    out["value"] = big["kikerax"]["decode_tok_s"]
    out["config"] = {"model": "Kikerax, (differential attention + dense, attention beside a recurrent unit + routed experts) x 2",
                     "global_batch": B, "seq_len": T, "parallelism": "single GPU", "l2": "weights of a step exceed the L2"}
    return out


def reference_arm_reason() -> str:
    """Why `--impl reference` has nothing to run, as found on this image (one line)."""
    return ("kurulav1/cpi is a CMake C++/CUDA project (no setup.py or pyproject.toml, so pip has nothing to install); "
            "its stock CMake build stops here at the first C++ file: CMakeLists.txt:40 passes '-Wall -Wextra -Wpedantic' "
            "as one unquoted generator expression and g++ gets the option '-Wpedantic>'; and its CUDA engine carries "
            "the 48-layer Scout sizes as compiled-in members (include/engine/llama4_cuda_engine.hpp:121-140) and runs "
            "one sequence, so it could run neither this 24-layer configuration nor a batch of 8 unmodified")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="cpi_b200")
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--sizes", default="", help="--workload nogapel | kikerax: a comma-separated subset of its size points")
    ap.add_argument("--workload", choices=["scout24", "maverick4", "long131k", "contexts", "cpu_baseline", "veredra", "savenex", "nogapel", "kikerax"],
                    default="scout24")
    ap.add_argument("--reference-root", default=os.environ.get("CPI_REFERENCE_ROOT"),
                    help="a checkout of kurulav1/cpi (for --workload cpu_baseline)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": reference_arm_reason()}))
        return 0
    if args.workload == "cpu_baseline":
        print(json.dumps(run_cpu_baseline(args)))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "cpi_b200 is a single-GPU library: run with --gpus 1", "n_gpus": args.gpus}))
        return 2
    args.warmup = max(args.warmup, 3)
    if args.workload == "veredra":
        print(json.dumps(run_veredra(args)))
        return 0
    if args.workload == "savenex":
        print(json.dumps(run_savenex(args)))
        return 0
    if args.workload == "kikerax":
        print(json.dumps(run_kikerax(args)))
        return 0
    if args.workload == "nogapel":
        print(json.dumps(run_nogapel(args)))
        return 0
    if args.workload == "contexts":
        print(json.dumps(run_contexts(args)))
        return 0
    print(json.dumps(run(args) if args.workload == "scout24" else run_workload(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
