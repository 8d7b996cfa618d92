"""Plain, slow implementation of Qwen2-MoE: whole sequences, no cache, one function per part, float64
arithmetic on the float32 (or bfloat16) weight values.  It runs where its tensors are: on the CPU for the tiny
models, and with float64 tensors on the GPU where a test holds the engine to it at real layer sizes.

It shares no code with the package: it reads ``config.json`` as a dict and the safetensors file
with a reader of its own.  Every function is written from the reference's formulas and cites
them (paths inside the reference project).  Where the reference leaves a configuration key
unread (``mlp_only_layers``, ``use_sliding_window``, ``max_window_layers``) the rule is the
one of the configuration format, stated at the function.

It was compared once with the reference's own CPU forward pass (tools/ref_top5.cpp, compiled
unchanged on this CPU) on tiny random models: see tests/golden/.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64


# ------------------------------------------------------------------------------ reading a folder
def read_folder(model_dir: str):
    """(config dict, {name: float64 tensor}) of a folder with config.json and *.safetensors
    (container layout: src/safetensors.cpp:12-53)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    for fn in sorted(os.listdir(model_dir)):
        if not fn.endswith(".safetensors"):
            continue
        with open(os.path.join(model_dir, fn), "rb") as f:
            raw = f.read()
        (n,) = struct.unpack("<Q", raw[:8])
        header = json.loads(raw[8:8 + n])
        for name, ent in header.items():
            if name == "__metadata__":
                continue
            b, e = ent["data_offsets"]
            buf = raw[8 + n + b:8 + n + e]
            dt = ent["dtype"]
            if dt == "BF16":  # widen exactly: bits << 16  (src/hip_ops.hip:34-36)
                u = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
                arr = u.view(np.float32).astype(np.float64)
            elif dt == "F32":
                arr = np.frombuffer(buf, dtype=np.float32).astype(np.float64)
            elif dt == "F16":
                arr = np.frombuffer(buf, dtype=np.float16).astype(np.float64)
            elif dt == "F64":
                arr = np.frombuffer(buf, dtype=np.float64).copy()
            else:
                raise ValueError(f"{name}: dtype {dt}")
            tensors[name] = torch.from_numpy(arr.copy()).reshape(ent["shape"])
    return cfg, tensors


# ------------------------------------------------------------------------------ configuration rules
def head_dim(cfg) -> int:
    """head_dim, or hidden_size / heads when absent (include/nanovllm/config.hpp:91-92)."""
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def layer_is_sparse(cfg, l: int) -> bool:
    """include/nanovllm/config.hpp:69, plus the format's ``mlp_only_layers`` (dense where listed)."""
    return (cfg.get("num_experts", 0) > 0 and l not in (cfg.get("mlp_only_layers") or [])
            and (l + 1) % cfg.get("decoder_sparse_step", 1) == 0)


def layer_window(cfg, l: int) -> int:
    """0 = every earlier key.  The format's rule: a window of ``sliding_window`` keys (the query's own
    position included) on layers ``l >= max_window_layers`` when ``use_sliding_window``; the key range
    is the one of the reference's windowed path (src/vulkan_model.cpp:786-789)."""
    if cfg.get("use_sliding_window", False) and cfg.get("sliding_window", 0) and l >= cfg.get("max_window_layers", 0):
        return int(cfg["sliding_window"])
    return 0


# ------------------------------------------------------------------------------ parts
def embedding(table, ids):
    """h[t] = table[id_t]  (src/hip_ops.hip:553-563)."""
    return table[torch.as_tensor(ids, dtype=torch.long, device=table.device)].clone()


def rms_norm(x, w, eps: float):
    """y = x * (1 / sqrt(mean(x^2) + eps)) * w  (tools/ref_top5.cpp:243-252; src/hip_ops.hip:403-416)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(ms + eps)) * w


def rope_neox(x, positions, theta: float):
    """x: [T, heads, D].  inv_freq[d] = float32(1 / theta^(2d/D)); angle = float32(pos) * inv_freq[d]
    in float32; pairs (d, d + D/2)  (tools/ref_top5.cpp:321-323, 401-420; src/hip_ops.hip:431-450)."""
    T, Hn, D = x.shape
    half = D // 2
    inv = np.array([1.0 / (theta ** ((2.0 * i) / D)) for i in range(half)], dtype=np.float64).astype(np.float32)
    pos = np.asarray(positions, dtype=np.float32)[:, None]
    ang = (pos * inv[None, :]).astype(np.float32)            # float32 product, as the reference
    c = torch.from_numpy(np.cos(ang.astype(np.float64)))[:, None, :].to(x.device)
    s = torch.from_numpy(np.sin(ang.astype(np.float64)))[:, None, :].to(x.device)
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def causal_attention(q, k, v, scale: float, window: int = 0):
    """q: [T, Hq, D]; k, v: [T, Hkv, D]; query head h reads kv head h // (Hq/Hkv); row t sees keys
    [max(0, t+1-window), t]; softmax of (q.k)*scale  (tools/ref_top5.cpp:425-455;
    src/hip_ops.hip:473-551)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    out = torch.zeros(T, Hq, D, dtype=F64, device=q.device)
    for h in range(Hq):
        kh = h // rep
        s = (q[:, h, :] @ k[:, kh, :].T) * scale                       # [T, T]
        i = torch.arange(T, device=q.device)[:, None]
        j = torch.arange(T, device=q.device)[None, :]
        keep = j <= i
        if window > 0:
            keep &= j >= i + 1 - window
        s = s.masked_fill(~keep, -float("inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def attention_layer(x_norm, W, prefix: str, cfg, l: int, positions):
    """q/k/v projections with bias, rotation, attention, output projection without bias
    (tools/ref_top5.cpp:344-463; src/model.cpp:764-786)."""
    T = x_norm.shape[0]
    Hq, Hkv, D = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"]), head_dim(cfg)

    def proj(name, heads):
        y = x_norm @ W[prefix + name + ".weight"].T
        if prefix + name + ".bias" in W:
            y = y + W[prefix + name + ".bias"]
        return y.reshape(T, heads, D)

    q, k, v = proj("q_proj", Hq), proj("k_proj", Hkv), proj("v_proj", Hkv)
    theta = float(cfg.get("rope_theta", 10000.0))
    q, k = rope_neox(q, positions, theta), rope_neox(k, positions, theta)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(D)))          # 1/sqrt(float(D)), src/model.cpp:710
    a = causal_attention(q, k, v, scale, layer_window(cfg, l))
    return a.reshape(T, Hq * D) @ W[prefix + "o_proj.weight"].T


def silu_mul(g, u):
    """g / (1 + exp(-g)) * u  (src/hip_ops.hip:419-429)."""
    return g / (1.0 + torch.exp(-g)) * u


def dense_mlp(x_norm, W, prefix: str):
    """down(silu(gate x) * up x)  (tools/ref_top5.cpp:554-584; src/model.cpp:828-832)."""
    g = x_norm @ W[prefix + "gate_proj.weight"].T
    u = x_norm @ W[prefix + "up_proj.weight"].T
    return silu_mul(g, u) @ W[prefix + "down_proj.weight"].T


def route(x_norm, Wg, top_k: int, renorm: bool, margins: list | None = None):
    """p = softmax(x Wg^T) over all experts; the top_k largest in descending order, a tie going to the
    lower index (selection with strict >); weights p or p / sum(p_topk)
    (tools/ref_top5.cpp:484-515; src/hip_ops.hip:813-841).  Returns (idx [T,K], w [T,K]).
    ``margins``, if a list, receives per row the gap between the top_k-th and the next router logit as a fraction
    of the spread of the row's logits (largest minus smallest): how far the row is from choosing another expert."""
    logits = (x_norm @ Wg.T).to(torch.float32).to(F64)                 # router logits are stored as float32
    p = torch.softmax(logits, dim=-1)
    T, E = p.shape
    idx = torch.zeros(T, top_k, dtype=torch.long, device=p.device)
    w = torch.zeros(T, top_k, dtype=F64, device=p.device)
    rem = p.clone()
    rows = torch.arange(T, device=p.device)
    for k in range(top_k):                  # one selection pass per rank; argmax returns the first largest
        best = torch.argmax(rem, dim=-1)
        idx[:, k], w[:, k] = best, rem[rows, best]
        rem[rows, best] = -1.0
    if margins is not None and top_k < E:
        top = torch.sort(logits, dim=-1, descending=True).values
        margins.append(((top[:, top_k - 1] - top[:, top_k]) / (top[:, 0] - top[:, -1]).clamp_min(1e-30)).cpu())
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return idx, w.to(torch.float32).to(F64)                            # weights are stored as float32


def sparse_mlp(x_norm, W, prefix: str, cfg, margins: list | None = None):
    """shared expert times its sigmoid gate, plus the routed experts
    (tools/ref_top5.cpp:467-552; src/model.cpp:789-827).  The reference walks a row's experts in rank order;
    here the rows of one expert are taken together (float64 sums: the order moves nothing that is compared)."""
    T, H = x_norm.shape
    E, K = cfg["num_experts"], cfg["num_experts_per_tok"]
    idx, w = route(x_norm, W[prefix + "gate.weight"], K, bool(cfg.get("norm_topk_prob", False)), margins)
    y = torch.zeros(T, H, dtype=F64, device=x_norm.device)
    if cfg.get("shared_expert_intermediate_size", 0) > 0:
        sh = dense_mlp(x_norm, W, prefix + "shared_expert.")
        gate = 1.0 / (1.0 + torch.exp(-(x_norm @ W[prefix + "shared_expert_gate.weight"].reshape(-1))))
        y = y + gate[:, None] * sh
    stacked = prefix + "experts.gate_up_proj" in W
    I = cfg["moe_intermediate_size"]
    for e in range(E):
        hit = (idx == e)
        rows = torch.nonzero(hit.any(dim=-1)).reshape(-1)
        if rows.numel() == 0:
            continue
        if stacked:      # [E, 2I, H] gate rows then up rows; [E, H, I]  (src/model.cpp:274-281, 356-365)
            gu, dn = W[prefix + "experts.gate_up_proj"][e], W[prefix + "experts.down_proj"][e]
            wg, wu = gu[:I], gu[I:]
        else:
            pe = f"{prefix}experts.{e}."
            wg, wu, dn = W[pe + "gate_proj.weight"], W[pe + "up_proj.weight"], W[pe + "down_proj.weight"]
        xe = x_norm[rows]
        out = silu_mul(xe @ wg.T, xe @ wu.T) @ dn.T
        we = (w[rows] * hit[rows]).sum(dim=-1)                          # an expert appears once in a row's top k
        y[rows] = y[rows] + we[:, None] * out
    return y


def forward(cfg, W, ids, positions=None, margins: list | None = None):
    """Logits [T, V] (float64) of one whole sequence  (tools/ref_top5.cpp:314-592;
    src/model.cpp:698-848).  x <- x + attention(norm(x)); x <- x + mlp(norm(x)); final norm; head.
    ``W`` is any mapping from tensor names to float64 tensors (all on one device); ``margins`` collects the
    router's margins of every sparse layer (see ``route``)."""
    T = len(ids)
    if positions is None:
        positions = list(range(T))
    eps = float(np.float32(cfg.get("rms_norm_eps", 1e-6)))             # eps cast to float, src/model.cpp:709
    x = embedding(W["model.embed_tokens.weight"], ids)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = rms_norm(x, W[p + "input_layernorm.weight"], eps)
        x = x + attention_layer(h, W, p + "self_attn.", cfg, l, positions)
        h = rms_norm(x, W[p + "post_attention_layernorm.weight"], eps)
        if layer_is_sparse(cfg, l):
            x = x + sparse_mlp(h, W, p + "mlp.", cfg, margins)
        else:
            x = x + dense_mlp(h, W, p + "mlp.")
    h = rms_norm(x, W["model.norm.weight"], eps)
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else W["lm_head.weight"]
    return h @ head.T


# ------------------------------------------------------------------------------ sampling
def sample(logits, temperature: float, u: float) -> int:
    """temperature <= 0: first largest logit; else p_i = exp((l_i - max)/T), target u * sum(p), first i
    whose running sum exceeds it, V-1 if none  (include/nanovllm/sampler.hpp:10-34)."""
    l = np.asarray(logits, dtype=np.float64)
    if temperature <= 0:
        return int(np.argmax(l))
    p = np.exp((l - l.max()) * (1.0 / temperature))
    target = u * p.sum()
    cum = np.cumsum(p)
    hit = np.nonzero(cum > target)[0]
    return int(hit[0]) if len(hit) else len(l) - 1


def sample_row(logits, temperature: float, top_p: float, u: float, recent=(), rep_penalty: float = 1.0,
               rep_window: int = 64) -> int:
    """The reference's second sampler (include/nanovllm/sampler.hpp:46-88): greedy at temperature <= 0, else
    s_i = float(exp((l_i - max) / T)); the ids seen among the last ``rep_window`` of ``recent`` (0: all of it; each
    id once) have s divided by float(rep_penalty); tokens in descending order of s (the reference's sort leaves
    the order of equal scores open: here the lower id first); the nucleus ends at the first place i > 0 whose
    running share reaches top_p; r = u * (share of the nucleus), answer = first token whose running share
    reaches r, else the nucleus's last."""
    l = np.asarray(logits, dtype=np.float32)
    V = len(l)
    if temperature <= 0:
        return int(np.argmax(l))
    mx = l.max()
    sc = np.exp((l - mx).astype(np.float64) / temperature).astype(np.float32)
    recent = list(recent)
    if rep_penalty != 1.0 and rep_penalty > 0.0 and recent:
        w = min(rep_window, len(recent)) if rep_window > 0 else len(recent)
        seen = []
        for tok in recent[len(recent) - w:]:
            if tok < 0 or tok >= V or tok in seen:
                continue
            seen.append(tok)
            sc[tok] = np.float32(sc[tok] / np.float32(rep_penalty))
    total = float(np.sum(sc.astype(np.float64)))
    order = np.argsort(-sc.astype(np.float64), kind="stable")
    share = sc[order].astype(np.float64) / total
    acc, keep = 0.0, V
    for i in range(V):
        acc += share[i]
        if acc >= top_p and i > 0:
            keep = i + 1
            break
    r, run = u * acc, 0.0
    for i in range(keep):
        run += share[i]
        if r <= run:
            return int(order[i])
    return int(order[keep - 1])


def greedy_generate(cfg, W, prompt, n_new: int):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]
