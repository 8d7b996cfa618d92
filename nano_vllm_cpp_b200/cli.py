"""The ``nanovllm`` command line, with the reference's options where it has them
(src/main.cpp:25-31, 343-365):

    nanovllm <model_dir> --tokens 1,2,3 [--max-tokens N] [--temperature T] [--max-model-len N]
                         [--num-kv-blocks N]
    nanovllm --bench <model_dir> [--num-seqs N] [--max-tokens N] [--max-model-len N]
    nanovllm --config config.json [--seed S] --tokens 1,2,3 ...      (random weights, no model folder)

The prompt is given as token ids (``--tokens``); this engine has no tokenizer, so a text prompt
is refused.  ``--chat`` and ``--server`` belong to parts of the reference that are not built
here.  ``--expert-budget`` is accepted and ignored: every expert stays resident in device memory.
``--top-p``, ``--rep-penalty`` and ``--rep-window`` are those of the reference's second command line
(src/main_vulkan.cpp:260-298): nucleus sampling, and the scores of ids among the last W completion tokens
divided by THETA (1.0 = off, W = 0: the whole completion).
``temperature``, ``top_p`` and ``max_new_tokens`` of the model folder's ``generation_config.json`` are the
defaults of the options that are not given (src/main_vulkan.cpp:360-363).
Exit codes as the reference's: 1 usage, 2 error (src/main.cpp:432-438).
"""
from __future__ import annotations

import sys
import time

USAGE = """Usage: nanovllm <model_dir> --tokens 1,2,3 [--max-tokens N] [--temperature T] [--max-model-len N]
       nanovllm --bench <model_dir> [--num-seqs N] [--max-tokens N] [--max-model-len N]
       nanovllm --config <config.json> [--seed S] --tokens 1,2,3 ...   (random weights, no model folder)
  further options: --num-kv-blocks N  --dtype bfloat16|float32 (or bf16|fp32)  --random-weights  --seed S
                   --page-size N  --prefill-chunk N  --max-num-batched-tokens N  --max-num-seqs N
                   --eos ID  --ignore-eos  --expert-budget GB (ignored)
                   --top-p P  --rep-penalty THETA  --rep-window W   (nucleus sampling and repetition penalty)
"""


def generation_defaults(model_dir: str) -> dict:
    """``temperature``, ``top_p`` and ``max_tokens`` (from ``max_new_tokens`` >= 1) of
    ``<model_dir>/generation_config.json``, read best-effort: a missing or unreadable file or key gives no
    default (include/nanovllm/config.hpp:213-250).  They stand in for options that the command line does not
    give (src/main_vulkan.cpp:360-363)."""
    import json
    import os
    out = {}
    try:
        with open(os.path.join(model_dir, "generation_config.json")) as f:
            g = json.load(f)
        if isinstance(g.get("temperature"), (int, float)) and not isinstance(g.get("temperature"), bool):
            out["temperature"] = float(g["temperature"])
        if isinstance(g.get("top_p"), (int, float)) and not isinstance(g.get("top_p"), bool):
            out["top_p"] = float(g["top_p"])
        if isinstance(g.get("max_new_tokens"), int) and not isinstance(g.get("max_new_tokens"), bool) \
                and g["max_new_tokens"] >= 1:
            out["max_tokens"] = int(g["max_new_tokens"])
    except (OSError, ValueError, AttributeError):
        return {}
    return out


def parse_ids(s: str) -> list:
    """``1,2,3`` -> [1, 2, 3]  (src/main.cpp:56-66)."""
    return [int(x) for x in s.split(",") if x.strip() != ""]


def main(argv=None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    if not args:
        sys.stderr.write(USAGE)
        return 1
    opt = dict(model_dir="", prompt="", prompt_ids=[], max_tokens=64, temperature=0.6, max_model_len=4096,
               bench=False, num_seqs=4, num_kv_blocks=0, dtype="bfloat16", random_weights=False, seed=0,
               page_size=16, prefill_chunk=0, max_num_batched_tokens=16384, max_num_seqs=512, eos=-1,
               ignore_eos=False, top_p=1.0, rep_penalty=1.0, rep_window=64, config="")
    with_value = {"--tokens": ("prompt_ids", parse_ids), "--max-tokens": ("max_tokens", int),
                  "--temperature": ("temperature", float), "--max-model-len": ("max_model_len", int),
                  "--num-kv-blocks": ("num_kv_blocks", int), "--expert-budget": (None, float),
                  "--num-seqs": ("num_seqs", int), "--dtype": ("dtype", str), "--seed": ("seed", int),
                  "--page-size": ("page_size", int), "--prefill-chunk": ("prefill_chunk", int),
                  "--max-num-batched-tokens": ("max_num_batched_tokens", int),
                  "--max-num-seqs": ("max_num_seqs", int), "--eos": ("eos", int), "--top-p": ("top_p", float),
                  "--rep-penalty": ("rep_penalty", float), "--rep-window": ("rep_window", int),
                  "--config": ("config", str)}
    i = 0
    given = set()
    try:
        while i < len(args):
            a = args[i]
            if a in with_value and i + 1 < len(args):
                key, conv = with_value[a]
                i += 1
                if key is not None:
                    opt[key] = conv(args[i])
                    given.add(key)
            elif a == "--bench":
                opt["bench"] = True
            elif a == "--random-weights":
                opt["random_weights"] = True
            elif a == "--ignore-eos":
                opt["ignore_eos"] = True
            elif a in ("--chat", "--server", "--host", "--port"):
                sys.stderr.write(f"Error: {a} belongs to the chat/server front ends, which this engine does not have\n")
                return 2
            elif a in ("--help", "-h"):
                sys.stderr.write(USAGE)
                return 0
            elif not opt["model_dir"]:
                opt["model_dir"] = a
            elif not opt["prompt"]:
                opt["prompt"] = a
            else:
                sys.stderr.write(USAGE)
                return 1
            i += 1
    except ValueError as e:
        sys.stderr.write(f"Error: bad option value: {e}\n")
        return 1
    if opt["config"] and opt["model_dir"] and not opt["prompt"]:
        # with --config there is no model folder: a positional argument is the (text) prompt
        opt["prompt"], opt["model_dir"] = opt["model_dir"], ""
    if not opt["model_dir"] and not opt["config"]:
        sys.stderr.write(USAGE)
        return 1
    for key, value in generation_defaults(opt["model_dir"]).items():
        if key not in given:                  # explicit options win
            opt[key] = value
    try:
        if opt["config"]:
            return _run_from_config(opt)
        return _run(opt)
    except Exception as e:  # src/main.cpp:432-438
        sys.stderr.write(f"Error: {e}\n")
        return 2


def _run_from_config(opt) -> int:
    """``--config <json>``: a run with random weights (drawn from ``--seed``) of the model that the file describes,
    without a model folder: the file becomes the ``config.json`` of a temporary one."""
    import os
    import shutil
    import tempfile
    with tempfile.TemporaryDirectory(prefix="nanovllm_config_") as d:
        shutil.copyfile(opt["config"], os.path.join(d, "config.json"))
        return _run(dict(opt, model_dir=d, random_weights=True))


def _run(opt) -> int:
    from .config import SamplingParams
    from .engine.llm_engine import LLMEngine
    if not opt["bench"] and not opt["prompt_ids"]:
        raise ValueError("give the prompt as token ids with --tokens 1,2,3 (this engine has no tokenizer)")
    engine = LLMEngine(opt["model_dir"], opt["max_model_len"], opt["num_kv_blocks"], dtype=opt["dtype"],
                       random_weights=opt["random_weights"], seed=opt["seed"], kvcache_block_size=opt["page_size"],
                       prefill_chunk=opt["prefill_chunk"], max_num_batched_tokens=opt["max_num_batched_tokens"],
                       max_num_seqs=opt["max_num_seqs"], eos=opt["eos"])
    sp = SamplingParams(temperature=opt["temperature"], max_tokens=opt["max_tokens"],
                        ignore_eos=opt["ignore_eos"] or opt["bench"], top_p=opt["top_p"],
                        repetition_penalty=opt["rep_penalty"], repetition_window=opt["rep_window"])
    if opt["bench"]:
        # synthetic prompts of 64 ids, 1 + ((i*37 + t) % (V-2))  (src/main.cpp:388-412)
        import torch
        span = max(1, engine.vocab_size - 2)
        for i in range(opt["num_seqs"]):
            engine.add_request([1 + ((i * 37 + t) % span) for t in range(64)], sp)
        pp_secs = tg_secs = 0.0
        pp_toks = gen = 0
        while not engine.is_finished():
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = engine.step()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            if out.num_prefill_tokens:
                pp_toks += out.num_prefill_tokens
                pp_secs += dt
            else:
                gen += out.num_decode_tokens
                tg_secs += dt
        print(f"total_seq: {opt['num_seqs']}  prompt_tokens: {pp_toks}  generated_tokens: {gen}")
        if pp_secs > 0:
            print(f"PP: {pp_toks} tokens / {pp_secs:.3f}s = {pp_toks / pp_secs:.1f} tok/s")
        if tg_secs > 0 and gen > 0:
            print(f"decode: {gen} tokens / {tg_secs:.3f}s = {gen / tg_secs:.1f} tok/s")
        return 0
    outs = engine.generate([opt["prompt_ids"]], [sp])
    for o in outs:
        print("token_ids: " + " ".join(str(t) for t in o["token_ids"]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
