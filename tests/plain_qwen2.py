"""A plain, slow Qwen2 forward pass for tests: whole sequences, no cache, one function per part.

Written from the formulas of the reference (KoduruChandrasekhar/TokenMill, paths below are within
that project) and sharing no code with ``tokenmill_b200``: it parses config.json itself, reads
safetensors itself and uses nothing but elementwise torch operations and matmul on the CPU. All
arithmetic is float32 (pass ``dtype=torch.float64`` to ``load_plain`` for a finer yardstick).

Weights are addressed by their checkpoint names (src/infer/model/loader.py:98-119).
"""

from __future__ import annotations

import glob
import json
from pathlib import Path

import torch


# --- model folder -------------------------------------------------------------------------------

def load_plain(folder, dtype=torch.float32):
    """(config dict, {checkpoint name: tensor}) of a model folder. Derived sizes follow
    src/infer/config.py:29-35,54-67."""
    from safetensors import safe_open

    folder = Path(folder)
    raw = json.loads((folder / "config.json").read_text())
    heads = raw["num_attention_heads"]
    theta = raw.get("rope_theta")
    if theta is None:
        theta = (raw.get("rope_parameters") or {}).get("rope_theta", 10000.0)
    cfg = {
        "vocab": raw["vocab_size"], "hidden": raw["hidden_size"], "inter": raw["intermediate_size"],
        "layers": raw["num_hidden_layers"], "heads": heads, "kv_heads": raw.get("num_key_value_heads", heads),
        "head_dim": raw.get("head_dim", raw["hidden_size"] // heads), "theta": float(theta),
        "eps": float(raw.get("rms_norm_eps", 1e-6)), "tied": bool(raw.get("tie_word_embeddings", False)),
    }
    weights = {}
    for file in sorted(glob.glob(str(folder / "*.safetensors"))):
        with safe_open(file, framework="pt", device="cpu") as f:
            for name in f.keys():
                weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights


# --- parts --------------------------------------------------------------------------------------

def plain_embedding(ids, table):
    """x = E[ids] (src/infer/model/qwen2.py:30,46)."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def plain_rmsnorm(x, weight, eps):
    """x * rsqrt(mean(x^2) + eps), then times the weight (src/infer/model/layers.py:41-44)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return weight * (x * torch.rsqrt(var + eps))


def plain_rope_tables(n_pos, head_dim, theta, dtype=torch.float32):
    """cos/sin tables [n_pos, head_dim] (src/infer/model/layers.py:47-52): inv_freq and the outer
    product in float32, the two halves of each row equal."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    freqs = torch.outer(torch.arange(n_pos).float(), inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def plain_rotate_half(x):
    """cat[-x[D/2:], x[:D/2]] (src/infer/model/layers.py:55-57)."""
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def plain_apply_rope(x, cos, sin, positions):
    """x [n, heads, D] at absolute positions [n] (src/infer/model/layers.py:60-64)."""
    pos = torch.as_tensor(positions, dtype=torch.long)
    c, s = cos[pos].unsqueeze(1), sin[pos].unsqueeze(1)
    return x * c + plain_rotate_half(x) * s


def plain_qkv(x, w, prefix, cfg):
    """Biased q/k/v projections reshaped to heads (src/infer/model/layers.py:139,143-147; the
    reference fuses the three matrices, rows [q; k; v], which is the same product)."""
    n = x.shape[0]
    q = x @ w[f"{prefix}.q_proj.weight"].T + w[f"{prefix}.q_proj.bias"]
    k = x @ w[f"{prefix}.k_proj.weight"].T + w[f"{prefix}.k_proj.bias"]
    v = x @ w[f"{prefix}.v_proj.weight"].T + w[f"{prefix}.v_proj.bias"]
    D = cfg["head_dim"]
    return q.view(n, cfg["heads"], D), k.view(n, cfg["kv_heads"], D), v.view(n, cfg["kv_heads"], D)


def plain_causal_attention(q, k, v, scale, window=None, q_positions=None):
    """q [nq, H, D] over keys k, v [nk, KVH, D]; query i sits at absolute position q_positions[i]
    (default: the last nq of the nk positions) and sees keys j <= its position, and j > position -
    window when a window is given. Scores, mask and softmax as the reference's explicit path
    (src/infer/model/layers.py:72-83); query head h reads kv head h // G (layers.py:86-97)."""
    nq, H, D = q.shape
    nk, KVH, _ = k.shape
    G = H // KVH
    if q_positions is None:
        q_positions = torch.arange(nk - nq, nk)
    qpos = torch.as_tensor(q_positions, dtype=torch.long)
    kpos = torch.arange(nk)
    mask = kpos[None, :] <= qpos[:, None]
    if window:
        mask &= kpos[None, :] > (qpos[:, None] - window)
    out = torch.empty_like(q)
    for h in range(H):
        scores = (q[:, h, :] @ k[:, h // G, :].T) * scale
        scores = scores.masked_fill(~mask, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h, :] = probs @ v[:, h // G, :]
    return out


def plain_attention_block(x, w, prefix, cfg, cos, sin, window=None):
    """projection -> rope -> causal attention -> output projection (src/infer/model/layers.py:142-150)."""
    n = x.shape[0]
    q, k, v = plain_qkv(x, w, prefix, cfg)
    pos = torch.arange(n)
    q, k = plain_apply_rope(q, cos, sin, pos), plain_apply_rope(k, cos, sin, pos)
    out = plain_causal_attention(q, k, v, cfg["head_dim"] ** -0.5, window=window)
    return out.reshape(n, cfg["heads"] * cfg["head_dim"]) @ w[f"{prefix}.o_proj.weight"].T


def plain_silu(x):
    return x / (1.0 + torch.exp(-x))


def plain_swiglu(x, w, prefix):
    """down(silu(gate(x)) * up(x)) (src/infer/model/layers.py:162-164)."""
    gate = x @ w[f"{prefix}.gate_proj.weight"].T
    up = x @ w[f"{prefix}.up_proj.weight"].T
    return (plain_silu(gate) * up) @ w[f"{prefix}.down_proj.weight"].T


def plain_decoder_layer(x, w, i, cfg, cos, sin):
    """x + attn(ln1(x)), then x + mlp(ln2(x)) (src/infer/model/qwen2.py:21-23)."""
    p = f"model.layers.{i}"
    x = x + plain_attention_block(plain_rmsnorm(x, w[f"{p}.input_layernorm.weight"], cfg["eps"]), w,
                                  f"{p}.self_attn", cfg, cos, sin)
    return x + plain_swiglu(plain_rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], cfg["eps"]), w, f"{p}.mlp")


def plain_hidden(cfg, w, ids):
    """Final-normed hidden states [n, hidden] of one whole sequence (src/infer/model/qwen2.py:43-49)."""
    dtype = w["model.embed_tokens.weight"].dtype
    cos, sin = plain_rope_tables(len(ids), cfg["head_dim"], cfg["theta"], dtype)
    x = plain_embedding(ids, w["model.embed_tokens.weight"])
    for i in range(cfg["layers"]):
        x = plain_decoder_layer(x, w, i, cfg, cos, sin)
    return plain_rmsnorm(x, w["model.norm.weight"], cfg["eps"])


def plain_logits(cfg, w, ids):
    """Logits [n, vocab] at every position of one whole sequence; the output matrix is the embedding
    when tied (src/infer/model/qwen2.py:39-41,51-52)."""
    out_w = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return plain_hidden(cfg, w, ids) @ out_w.T


def plain_greedy(cfg, w, prompt, n_new):
    """Greedy continuation by recomputing the whole sequence for every token; argmax takes the
    lowest index on ties (src/infer/sampling.py:30, src/infer/model/qwen2.py:85-106)."""
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(plain_logits(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt):]


# --- sampling -----------------------------------------------------------------------------------

def plain_filtered_probs(logits, temperature, top_k=-1, top_p=1.0):
    """Probabilities the reference samples from (src/infer/sampling.py:12-25,35-42): logits / T, keep
    the top_k largest, softmax, drop a token once the mass ranked before it exceeds top_p (the first
    always stays), softmax over what is left. logits [V] -> probs [V] float64."""
    z = logits.double() / temperature
    V = z.numel()
    if (top_k and top_k > 0) or top_p < 1.0:
        sorted_z, idx = z.sort(descending=True)
        k = V if not top_k or top_k <= 0 else min(top_k, V)
        remove = torch.arange(V) >= k
        probs = sorted_z.masked_fill(remove, float("-inf")).softmax(-1)
        cum = probs.cumsum(-1)
        remove |= (cum - probs) > top_p
        remove[0] = False
        sorted_z = sorted_z.masked_fill(remove, float("-inf"))
        z = torch.empty_like(z).scatter_(0, idx, sorted_z)
    return z.softmax(-1)


def plain_inverse_cdf(probs, u):
    """First index whose running sum of probabilities exceeds u (vocabulary order)."""
    cdf = probs.double().cumsum(0)
    target = u * float(cdf[-1])
    i = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True))
    return min(i, probs.numel() - 1)


def tolerance(reference: torch.Tensor, dtype: str) -> float:
    """Largest absolute logit difference the tests accept against the plain float32 result:
    a fraction of the largest logit magnitude (random weights give logits well below 1)."""
    scale = float(reference.abs().max())
    return (2e-4 if dtype == "float32" else 3e-2) * scale


