"""Makes tests/golden/ref_top5.json: what the reference's own CPU forward pass
(tools/ref_top5.cpp, compiled unchanged with g++) prints for tiny random Qwen2-MoE models.

    python tests/golden/make_golden.py /path/to/reference

For each case it writes a model folder into a temporary directory with ``tiny_model`` below
(numpy's frozen RandomState stream, values rounded to bfloat16 and stored as BF16; the
reference reads matrices only as F16/BF16: src/safetensors.cpp:106-123), runs
``REF_MODEL=<dir> REF_TOKENS=<ids> ./ref_top5`` and records the top-5 ids and logits of the last
position and the routed experts of the last token per sparse layer.  The reference knows
neither ``mlp_only_layers`` nor windows, so case B lists a layer in ``mlp_only_layers`` only
where the step rule makes it dense anyway and keeps its prompts within the window.

tests/test_plain_vs_reference.py rebuilds the same folders and compares tests/plain_model.py
with the recorded output.
"""
import json
import os
import re
import struct
import subprocess
import sys
import tempfile

import numpy as np

CASES = {
    "A": dict(
        config=dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=2,
                    hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_experts=8,
                    num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=96,
                    intermediate_size=128, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True,
                    vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=128,
                    use_sliding_window=False, tie_word_embeddings=False, qkv_bias=True, hidden_act="silu"),
        seed=0, std=0.02, norm_std=0.0, prompts={"p5": 5, "p17": 17, "p33": 33}),
    "B": dict(
        config=dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=3,
                    hidden_size=96, num_attention_heads=3, num_key_value_heads=1, head_dim=32, num_experts=6,
                    num_experts_per_tok=3, moe_intermediate_size=48, shared_expert_intermediate_size=64,
                    intermediate_size=160, decoder_sparse_step=2, mlp_only_layers=[2], norm_topk_prob=False,
                    vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5, max_position_embeddings=256,
                    use_sliding_window=True, sliding_window=16, max_window_layers=1, tie_word_embeddings=True,
                    qkv_bias=True, hidden_act="silu"),
        seed=1, std=0.05, norm_std=0.1, prompts={"p1": 1, "p9": 9, "p16": 16}),
}


def to_bf16_bits(a):
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)   # round to nearest even


def tensor_names(cfg):
    H, V = cfg["hidden_size"], cfg["vocab_size"]
    D = cfg["head_dim"]
    q, kv = cfg["num_attention_heads"] * D, cfg["num_key_value_heads"] * D
    out = [("model.embed_tokens.weight", (V, H), "w")]
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        out += [(p + "input_layernorm.weight", (H,), "n"), (p + "post_attention_layernorm.weight", (H,), "n"),
                (p + "self_attn.q_proj.weight", (q, H), "w"), (p + "self_attn.q_proj.bias", (q,), "w"),
                (p + "self_attn.k_proj.weight", (kv, H), "w"), (p + "self_attn.k_proj.bias", (kv,), "w"),
                (p + "self_attn.v_proj.weight", (kv, H), "w"), (p + "self_attn.v_proj.bias", (kv,), "w"),
                (p + "self_attn.o_proj.weight", (H, q), "w")]
        sparse = (cfg["num_experts"] > 0 and l not in cfg["mlp_only_layers"]
                  and (l + 1) % cfg["decoder_sparse_step"] == 0)
        if sparse:
            I, SI = cfg["moe_intermediate_size"], cfg["shared_expert_intermediate_size"]
            out.append((p + "mlp.gate.weight", (cfg["num_experts"], H), "w"))
            for e in range(cfg["num_experts"]):
                pe = f"{p}mlp.experts.{e}."
                out += [(pe + "gate_proj.weight", (I, H), "w"), (pe + "up_proj.weight", (I, H), "w"),
                        (pe + "down_proj.weight", (H, I), "w")]
            out += [(p + "mlp.shared_expert.gate_proj.weight", (SI, H), "w"),
                    (p + "mlp.shared_expert.up_proj.weight", (SI, H), "w"),
                    (p + "mlp.shared_expert.down_proj.weight", (H, SI), "w"),
                    (p + "mlp.shared_expert_gate.weight", (1, H), "w")]
        else:
            I = cfg["intermediate_size"]
            out += [(p + "mlp.gate_proj.weight", (I, H), "w"), (p + "mlp.up_proj.weight", (I, H), "w"),
                    (p + "mlp.down_proj.weight", (H, I), "w")]
    out.append(("model.norm.weight", (H,), "n"))
    if not cfg["tie_word_embeddings"]:
        out.append(("lm_head.weight", (V, H), "w"))
    return out


def tiny_model(case, out_dir):
    """Writes config.json + model.safetensors (BF16) of a case; deterministic."""
    cfg = case["config"]
    rs = np.random.RandomState(case["seed"])
    header, blobs, off = {}, [], 0
    for name, shape, kind in tensor_names(cfg):
        z = rs.standard_normal(shape)
        a = z * case["std"] if kind == "w" else 1.0 + z * case["norm_std"]
        raw = to_bf16_bits(a).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return out_dir


def prompt_ids(case_name, n, vocab):
    rs = np.random.RandomState(1000 + ord(case_name) * 100 + n)
    return [int(x) for x in rs.randint(0, vocab, size=n)]


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/reference  (a checkout of Maxritz/Nano_vLLM_cpp)")
    ref = sys.argv[1]
    work = tempfile.mkdtemp()
    exe = os.path.join(work, "ref_top5")
    subprocess.check_call(["g++", "-std=c++20", "-O2", f"-I{ref}/include", f"{ref}/tools/ref_top5.cpp",
                           f"{ref}/src/gguf.cpp", f"{ref}/src/safetensors.cpp", f"{ref}/src/tokenizer.cpp",
                           "-o", exe])
    result = {}
    for cname, case in CASES.items():
        mdir = tiny_model(case, os.path.join(work, cname))
        for pname, n in case["prompts"].items():
            ids = prompt_ids(cname, n, case["config"]["vocab_size"])
            env = dict(os.environ, REF_MODEL=mdir, REF_TOKENS=",".join(map(str, ids)))
            r = subprocess.run([exe], env=env, capture_output=True, text=True, check=True)
            top = re.findall(r"(\d+)\((-?[\d.]+)\)", r.stdout.split("ref top5:")[1])
            routes = {}
            for m in re.finditer(r"REF route L(\d+) last:(.*)", r.stderr):
                routes[m.group(1)] = [[int(a), float(b)] for a, b in re.findall(r"(\d+)\((-?[\d.]+)\)", m.group(2))]
            result[f"{cname}/{pname}"] = {"ids": ids, "top5": [[int(a), float(b)] for a, b in top], "routes": routes}
            print(cname, pname, r.stdout.strip())
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_top5.json"), "w") as f:
        json.dump(result, f, indent=1)


if __name__ == "__main__":
    main()
