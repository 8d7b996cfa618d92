#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of the Qwen1.5-MoE-A2.7B shape with random bfloat16 weights, a batch
of 8 sequences each at a 2,048-token context; a step is one decode step of that batch.  ``value``
is decoded tokens per second timed on the device; ``e2e`` is the same through
``LLMEngine.step`` with host token ids in and out; ``prefill`` times one 2,048-token prompt;
``points`` holds decode at batch 1 and 64 and a mixed step (64 single rows beside a 512-token portion of a
prompt); ``roofline`` compares the bytes a decode step has to read (every weight it uses once, the cache of
the live requests) with the measured copy bandwidth.  A decode step here is the whole step: the model, the
sampling kernel behind it, and the next step reading the drawn tokens on the device.

``kernels`` (``--no-kernel-times`` leaves it out): per kernel class of one decode step and of the prompt, CUDA-event time,
calls and the fraction of the measured peak its bytes (decode) or flops (prompt) come to.  Those steps run
outside CUDA graphs with an event between any two kernels, one kernel after the other on one stream (the decode
step behind a delay kernel, so that the host has queued it all before the GPU starts): nothing overlaps, and
their sum is more than the step's own time.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(  # Qwen1.5-MoE-A2.7B layer sizes
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=24, hidden_size=2048,
    num_attention_heads=16, num_key_value_heads=16, head_dim=128, num_experts=60, num_experts_per_tok=4,
    moe_intermediate_size=1408, shared_expert_intermediate_size=5632, intermediate_size=5632,
    decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=False, vocab_size=151936, rope_theta=1000000.0,
    rms_norm_eps=1e-6, max_position_embeddings=8192, use_sliding_window=False, tie_word_embeddings=False,
    qkv_bias=True)
FULL_LAYERS = 24
SEED = 2
# A second shape for measurements beyond the default run (--shape 57b): the layer sizes of Qwen2-57B-A14B.
SHAPES = {
    "a2.7b": ("Qwen1.5-MoE-A2.7B shape", MODEL, FULL_LAYERS, SEED),
    "57b": ("Qwen2-57B-A14B shape", dict(
        MODEL, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
        num_experts=64, num_experts_per_tok=8, moe_intermediate_size=2560, shared_expert_intermediate_size=20480,
        intermediate_size=18944, max_position_embeddings=32768), 28, 4),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
MIXED_ROWS, MIXED_PORTION = 64, 512      # the mixed point: this many single rows beside a portion of this many tokens


def peaks():
    p = dict(FALLBACK_PEAKS)
    src = "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if k in m and isinstance(m[k], (int, float)):
                p[k] = float(m[k])
        src = "measured"
    except (OSError, ValueError):
        pass
    return p, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = max((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), default=None)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": reasons}


def weight_bytes(cfg, layers, distinct_experts):
    """Bytes of bf16 weights one decode step has to read: every matrix it uses, once."""
    H, D = cfg["hidden_size"], cfg["head_dim"]
    q, kv = cfg["num_attention_heads"] * D, cfg["num_key_value_heads"] * D
    I, SI, E = cfg["moe_intermediate_size"], cfg["shared_expert_intermediate_size"], cfg["num_experts"]
    per_layer = (q + 2 * kv) * H + H * q + E * H + 3 * SI * H + H
    total = layers * per_layer * 2 + sum(distinct_experts) * 3 * I * H * 2
    total += cfg["vocab_size"] * H * 2          # lm_head (the embedding rows read are negligible)
    return total


def kv_bytes(cfg, layers, contexts):
    return sum(contexts) * layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, layers, T):
    H, D = cfg["hidden_size"], cfg["head_dim"]
    q, kv = cfg["num_attention_heads"] * D, cfg["num_key_value_heads"] * D
    I, SI, E, K = (cfg["moe_intermediate_size"], cfg["shared_expert_intermediate_size"], cfg["num_experts"],
                   cfg["num_experts_per_tok"])
    per_tok = 2 * ((q + 2 * kv) * H + H * q + E * H + 3 * SI * H + H + K * 3 * I * H)
    attn = 4 * cfg["num_attention_heads"] * D * (T * (T + 1) // 2)       # causal QK^T and PV
    return layers * (per_tok * T + attn) + 2 * cfg["vocab_size"] * H


def kernel_times(runner, cfg, args, P, fill_context, StepEntry, ops, torch, g, V):
    """Per kernel class: CUDA-event time of one decode step at the default batch and of the prompt, run outside
    CUDA graphs.  What each class must move or compute comes from the launcher where it knows it (dense products) and
    from the configuration otherwise (attention, expert products)."""
    L, H, D = args.layers, cfg["hidden_size"], cfg["head_dim"]
    I, E, K = cfg["moe_intermediate_size"], cfg["num_experts"], cfg["num_experts_per_tok"]
    C = cfg["shared_expert_intermediate_size"] // I
    graphs, runner.cuda_graphs = runner.cuda_graphs, False
    out = []

    def rows_of(kt, steps, what, flops_of, bytes_of):
        for r in kt.summary()[:7]:
            ms = r["ms"] / steps
            nb = bytes_of(r) / steps
            fl = flops_of(r) / steps
            row = {"step": what, "name": r["name"], "calls": r["calls"] // steps, "ms": round(ms, 4)}
            if what == "decode" and nb:
                row["frac_hbm"] = round(nb / (ms * 1e-3) / (P["hbm_gbs"] * 1e9), 3)
            if what == "prefill" and fl:
                row["frac_bf16"] = round(fl / (ms * 1e-3) / (P["bf16_tflops"] * 1e12), 3)
            out.append(row)

    try:
        B = args.batch
        rids = fill_context(B)
        toks = torch.randint(0, V, (B,), generator=g).tolist()
        entries = [StepEntry(r, [t], [0]) for r, t in zip(rids, toks)]
        for _ in range(3):
            runner.step(entries, check=False)
        steps = 4
        with ops.KernelTimes() as kt:
            for _ in range(steps):
                ops.delay(30000)       # the host queues the whole step meanwhile: no waits for it between the kernels
                runner.step(entries, check=False)
        ctx_tokens = sum(runner.num_cached(r) for r in rids)
        distinct = [int((p.last_alignment.counts[:E] > 0).sum()) for p in
                    (l.feed_forward for l in runner.model.layers) if getattr(p, "last_alignment", None) is not None]
        per_layer_experts = (sum(distinct) / max(1, len(distinct)) + C) * steps * L

        def dec_bytes(r):
            if r["name"] == "attention_decode":
                return steps * L * ctx_tokens * 2 * cfg["num_key_value_heads"] * D * 2
            if r["name"].startswith("tc_gemm_grouped"):
                n = int(r["name"].split("N=")[1].split()[0])
                return per_layer_experts * n * (H if n == 2 * I else I) * 2
            return r["bytes"]

        rows_of(kt, steps, "decode", lambda r: 0.0, dec_bytes)
        for r in rids:
            runner.close(r)
        T = args.prefill_tokens
        ids = torch.randint(0, V, (T,), generator=g).tolist()
        for _ in range(2):
            runner.step([StepEntry("kt", ids, [T - 1])], check=False)
            runner.close("kt")
        with ops.KernelTimes() as kt:
            runner.step([StepEntry("kt", ids, [T - 1])], check=False)
        runner.close("kt")

        def pf_flops(r):
            if r["name"].startswith("attention_prefill"):
                return L * 4 * cfg["num_attention_heads"] * D * (T * (T + 1) // 2)
            if r["name"].startswith("tc_gemm_grouped"):
                n = int(r["name"].split("N=")[1].split()[0])
                return L * 2.0 * T * (K + C) * n * (H if n == 2 * I else I)
            return r["flops"]

        rows_of(kt, 1, "prefill", pf_flops, lambda r: 0.0)
    finally:
        runner.cuda_graphs = graphs
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--shape", default="a2.7b", choices=sorted(SHAPES), help="layer sizes (default: the headline shape)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-kernel-times", action="store_true", help="skip the per-kernel-class CUDA-event times")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "Maxritz/Nano_vLLM_cpp is a C++/CMake project, not installable with pip (no setup.py or "
                          "pyproject.toml), and its engine runs only on ROCm/HIP or Vulkan, which a B200 box has not"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from nano_vllm_cpp_b200.csrc import ops
    from nano_vllm_cpp_b200.engine.batch import StepEntry
    from nano_vllm_cpp_b200.engine.llm_engine import LLMEngine
    from nano_vllm_cpp_b200.config import SamplingParams

    shape_name, model, full_layers, seed = SHAPES[args.shape]
    if args.layers is None:
        args.layers = full_layers
    cfg = dict(model, num_hidden_layers=args.layers)
    P, peak_src = peaks()
    work = tempfile.mkdtemp(prefix="bench_model_")
    with open(os.path.join(work, "config.json"), "w") as f:
        json.dump(cfg, f)

    biggest = max(args.batch, 1 if args.no_points else 64)
    margin = args.steps + args.warmup + 80
    need_tokens = biggest * (args.context + margin) + args.prefill_tokens + MIXED_PORTION + 128
    page = 16
    # A run that would not fit comfortably is refused before anything is allocated (the full 57B shape holds
    # 115 GB of weights: give it fewer --layers, which the line then names beside the full number).
    H, D = cfg["hidden_size"], cfg["head_dim"]
    per_layer = ((cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * D * H + H * cfg["num_attention_heads"] * D
                 + cfg["num_experts"] * (H + 3 * cfg["moe_intermediate_size"] * H)
                 + 3 * cfg["shared_expert_intermediate_size"] * H + 3 * H)
    need_bytes = 2 * (args.layers * per_layer + 2 * cfg["vocab_size"] * H) + kv_bytes(cfg, args.layers, [need_tokens])
    free_bytes, _ = torch.cuda.mem_get_info()
    if need_bytes > 0.85 * free_bytes:
        print(f"bench.py: this run needs about {need_bytes / 1e9:.0f} GB of device memory and {free_bytes / 1e9:.0f} GB "
              f"are free; run it with fewer --layers (now {args.layers})")
        return 2
    eng = LLMEngine(work, max_model_len=max(args.context + margin, args.prefill_tokens) + 16, num_kv_blocks=(need_tokens + page - 1) // page,
                    dtype="bfloat16", random_weights=True, seed=seed, max_num_seqs=biggest + 1,
                    max_num_batched_tokens=max(args.prefill_tokens, biggest), enable_prefix_caching=False)
    runner = eng.runner
    dev = runner.device
    V = cfg["vocab_size"]
    g = torch.Generator().manual_seed(seed)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ------------------------------------------------------------------ prefill of one prompt
    prefill = None
    if not args.no_prefill:
        T = args.prefill_tokens
        ids = torch.randint(0, V, (T,), generator=g).tolist()
        times = []
        for it in range(args.warmup + 3):
            torch.cuda.synchronize()
            a, b = ev(), ev()
            a.record()
            runner.step([StepEntry("pf", ids, [T - 1])])
            b.record()
            torch.cuda.synchronize()
            runner.close("pf")
            if it >= args.warmup:
                times.append(a.elapsed_time(b))
        ms = sorted(times)[len(times) // 2]
        fl = prefill_flops(cfg, args.layers, T)
        prefill = {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3),
                   "frac": round(fl / (ms * 1e-3) / (P["bf16_tflops"] * 1e12), 4)}

    # ------------------------------------------------------------------ decode at a given batch
    def fill_context(B):
        """B requests whose caches hold `context` tokens of synthetic keys and values."""
        rids = [f"d{B}_{i}" for i in range(B)]
        for rid in rids:
            runner.open(rid)
            runner.manager.extend(rid, 0, args.context)
            runner.manager.commit(rid, args.context)
        for v in runner.cache.views:
            if v.kind == "kv" and v.write:
                v.k.normal_(0, 0.5)
                v.v.normal_(0, 0.5)
        return rids

    def moe_parts():
        return [l.feed_forward for l in runner.model.layers if hasattr(l.feed_forward, "last_alignment")]

    def decode_device(B, steps, warmup):
        """Whole decode steps: model, sampling kernel, and the next step's ids read from the tokens just drawn."""
        rids = fill_context(B)
        toks = torch.randint(0, V, (B,), generator=g).tolist()
        temps, us = [0.0] * B, [0.0] * B
        launches0 = 0
        a, b = ev(), ev()
        handle = None
        for it in range(warmup + steps):
            if it == warmup:
                torch.cuda.synchronize()
                launches0 = ops.launch_count()
                a.record()
            ids = toks if it == 0 else [-(r + 1) for r in range(B)]      # row r reads the token drawn for row r
            handle = runner.launch_tokens([StepEntry(r, [t], [0]) for r, t in zip(rids, ids)], temps, us)
        b.record()
        torch.cuda.synchronize()
        launches = ops.launch_count() - launches0
        runner.collect(handle)
        runner.ctx.err.check("decode")
        ms = a.elapsed_time(b) / steps
        distinct = [int((p.last_alignment.counts[:cfg["num_experts"]] > 0).sum()) for p in moe_parts()
                    if p.last_alignment is not None]
        ctxs = [runner.num_cached(r) for r in rids]
        for r in rids:
            runner.close(r)
        return ms, launches, distinct, ctxs

    def mixed_device(steps, warmup):
        """MIXED_ROWS single rows at the decode context beside the first MIXED_PORTION tokens of a new prompt."""
        rids = fill_context(MIXED_ROWS)
        toks = torch.randint(0, V, (MIXED_ROWS,), generator=g).tolist()
        portion = torch.randint(0, V, (MIXED_PORTION,), generator=g).tolist()
        a, b = ev(), ev()
        for it in range(warmup + steps):
            if it == warmup:
                torch.cuda.synchronize()
                a.record()
            entries = [StepEntry(r, [t], [0]) for r, t in zip(rids, toks)]
            entries.append(StepEntry(f"mx{it}", portion, [MIXED_PORTION - 1]))
            runner.step(entries, check=False)
            runner.close(f"mx{it}")
        b.record()
        torch.cuda.synchronize()
        runner.ctx.err.check("mixed step")
        ms = a.elapsed_time(b) / steps
        distinct = [int((p.last_alignment.counts[:cfg["num_experts"]] > 0).sum()) for p in moe_parts()
                    if p.last_alignment is not None]
        ctxs = [runner.num_cached(r) for r in rids]
        for r in rids:
            runner.close(r)
        # the portion alone, for comparison
        c, d = ev(), ev()
        for it in range(warmup + steps):
            if it == warmup:
                torch.cuda.synchronize()
                c.record()
            runner.step([StepEntry("mxa", portion, [MIXED_PORTION - 1])], check=False)
            runner.close("mxa")
        d.record()
        torch.cuda.synchronize()
        return ms, c.elapsed_time(d) / steps, distinct, ctxs

    clocks = ClockSampler()
    clocks.start()
    ms, launches, distinct, ctxs = decode_device(args.batch, args.steps, args.warmup)
    clk = clocks.stop()
    value = args.batch / ms * 1e3
    rbytes = weight_bytes(cfg, args.layers, distinct) + kv_bytes(cfg, args.layers, ctxs)
    achieved = rbytes / (ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": P["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / P["hbm_gbs"], 4), "of": peak_src,
                "bytes_per_step": rbytes, "distinct_experts_per_layer": round(sum(distinct) / max(1, len(distinct)), 1)}

    # ------------------------------------------------------------------ end to end through LLMEngine.step
    e2e = None
    if not args.no_e2e:
        # B requests with prompts of `context` tokens go through the public entry point: the engine runs their
        # prompts first (untimed), then every step decodes one token of each; host token ids in and out.
        B = args.batch
        sp = SamplingParams(temperature=0.0, max_tokens=args.steps + args.warmup + 24, ignore_eos=True)
        for _ in range(B):
            eng.add_request(torch.randint(0, V, (args.context,), generator=g).tolist(), sp)
        for _ in range(200):                  # until every request decodes
            out = eng.step()
            if out.num_decode_tokens == B and out.num_prefill_tokens == 0:
                break
        else:
            raise RuntimeError("bench.py: the requests of the end-to-end run never all reached decoding")
        for _ in range(args.warmup):
            eng.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n = 0
        for _ in range(args.steps):
            out = eng.step()
            n += len(out.new_tokens)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        e2e = {"value": round(n / dt, 1), "unit": "tokens/s", "h2d_bytes_per_step": eng.runner.last_h2d_bytes,
               "d2h_bytes_per_step": B * 4 + 4}
        while not eng.is_finished():      # let them run out (a few more steps)
            eng.step()

    points, mixed = {}, None
    if not args.no_points:
        ms_b64 = None
        for B in (1, 64):
            pms, _, pdistinct, pctxs = decode_device(B, max(8, args.steps // 2), args.warmup)
            points[f"decode_b{B}"] = round(B / pms * 1e3, 1)
            pbytes = weight_bytes(cfg, args.layers, pdistinct) + kv_bytes(cfg, args.layers, pctxs)
            points[f"decode_b{B}_frac"] = round(pbytes / (pms * 1e-3) / 1e9 / P["hbm_gbs"], 4)
            ms_b64 = pms
        mms, portion_ms, mdistinct, mctxs = mixed_device(max(6, args.steps // 4), args.warmup)
        mbytes = weight_bytes(cfg, args.layers, mdistinct) + kv_bytes(cfg, args.layers, mctxs)
        mflops = prefill_flops(cfg, args.layers, MIXED_PORTION)
        # the step can be no faster than its reads and no faster than its products: the larger of the two times
        floor_ms = max(mbytes / (P["hbm_gbs"] * 1e9), mflops / (P["bf16_tflops"] * 1e12)) * 1e3
        points["mixed_b64_p512"] = round((MIXED_ROWS + MIXED_PORTION) / mms * 1e3, 1)
        mixed = {"rows": MIXED_ROWS, "portion": MIXED_PORTION, "ms": round(mms, 3), "decode_b64_ms": round(ms_b64, 3),
                 "portion_alone_ms": round(portion_ms, 3), "frac": round(floor_ms / mms, 4),
                 "bound": "max(hbm bytes, bf16 flops)"}

    kernels = None
    if not args.no_kernel_times:
        kernels = kernel_times(runner, cfg, args, P, fill_context, StepEntry, ops, torch, g, V)

    line = {
        "metric": f"decode tok/s (batch {args.batch}, {args.context:,}-token context); "
                  f"prefill tok/s at {args.prefill_tokens:,} tokens; % of roofline",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": f"synthetic: random weights N(0,0.02) seed {seed}, uniform-random token ids, "
                                 "synthetic cache contents for the decode context",
        "config": {"model": shape_name, "global_batch": args.batch, "seq_len": args.context,
                   "parallelism": "single GPU", "num_hidden_layers": args.layers, "full_num_hidden_layers": full_layers,
                   "hidden_size": cfg["hidden_size"], "num_attention_heads": cfg["num_attention_heads"],
                   "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "num_experts": cfg["num_experts"], "num_experts_per_tok": cfg["num_experts_per_tok"],
                   "moe_intermediate_size": cfg["moe_intermediate_size"],
                   "shared_expert_intermediate_size": cfg["shared_expert_intermediate_size"],
                   "vocab_size": cfg["vocab_size"], "page_size": page, "prefill_tokens": args.prefill_tokens,
                   "l2": "inputs larger than L2 (weights and cache read per step exceed 126 MB)",
                   "step": "model + sampling kernel; ids fed back on the device"},
        "clocks": clk, "gpu_launches": launches, "roofline": roofline,
    }
    if prefill is not None:
        line["prefill"] = prefill
    if points:
        line["points"] = points
    if mixed is not None:
        line["mixed"] = mixed
    if kernels is not None:
        line["kernels"] = kernels
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
