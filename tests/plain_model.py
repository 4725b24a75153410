"""A plain, slow implementation of Qwen2-MoE for whole sequences: the tests' oracle.

It rests on the reference's formulas, not on its code run: the reference's model code is
HIP for gfx906 with rocBLAS (src/models/model.hip, src/ops/*.hip) and cannot be compiled
or imported on a machine without ROCm, so nothing here was compared with its output.
Each function cites the lines whose arithmetic it restates.  Where Qwen2-MoE needs what
the reference lacks (q/k/v bias, ``norm_topk_prob=false``, the shared expert with its
sigmoid gate, ``decoder_sparse_step`` / ``mlp_only_layers``, the sliding window), the
function says so.

No cache, no batching, no paging: one request, all its tokens at once, one function per
part.  It shares no code with the package under test: it reads config.json as a plain
dictionary and the weights through the `safetensors` package.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import numpy as np
import torch


# ---- reading a model folder -------------------------------------------------------------

def read_model_folder(model_dir: str, dtype: torch.dtype = torch.float32):
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights


# ---- random weights from a seed, without a file -------------------------------------------

def plain_random_tensor(seed: int, name: str, shape, init: str, device="cpu") -> torch.Tensor:
    """The engine's random-weights function restated (the reference has no such mode): element
    i of tensor `name` is made from (seed, name, i) alone.

        k1, k2 = first two little-endian 32-bit words of SHA-256("<seed>:<name>")
        mix(x) = x ^= x >> 16; x *= 0x7feb352d; x ^= x >> 15; x *= 0x846ca68b; x ^= x >> 16  (mod 2^32)
        s = mix(mix(lo32(i) ^ k1) ^ hi32(i) ^ k2)
        n = sum over c in (0x9e3779b9, 0x85ebca6b, 0xc2b2ae35, 0x27d4eb2f) of the three 10-bit
            fields of mix(s ^ c), minus 6138
        z = float32(n) * float32(1 / sqrt(1048575))
        value = bfloat16(0.02 * z) for "linear", bfloat16(1 + 0.05 * z) for "norm"

    Written with 64-bit torch integers holding 32-bit values (products are taken in two
    16-bit halves so that nothing overflows); runs on any torch device."""
    import hashlib
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    k1, k2 = int.from_bytes(digest[0:4], "little"), int.from_bytes(digest[4:8], "little")
    mask = (1 << 32) - 1

    def times(x, c):
        low = (x % 65536) * c
        high = ((x // 65536) * c) % 65536
        return (low + high * 65536) % (1 << 32)

    def mix(x):
        x = x ^ (x // 65536)
        x = times(x, 0x7FEB352D)
        x = x ^ (x // 32768)
        x = times(x, 0x846CA68B)
        return x ^ (x // 65536)

    count = 1
    for d in shape:
        count *= int(d)
    out = torch.empty(count, dtype=torch.float32, device=device)
    step = 1 << 24
    for a in range(0, count, step):
        i = torch.arange(a, min(count, a + step), dtype=torch.int64, device=device)
        s = mix(mix((i & mask) ^ k1) ^ (i // (1 << 32)) ^ k2)
        n = torch.zeros_like(s) - 6138
        for c in (0x9E3779B9, 0x85EBCA6B, 0xC2B2AE35, 0x27D4EB2F):
            w = mix(s ^ c)
            n = n + (w % 1024) + ((w // 1024) % 1024) + ((w // 1048576) % 1024)
        z = n.to(torch.float32) * float(np.float32(1.0 / math.sqrt(1048575.0)))
        v = (z * float(np.float32(0.05)) + 1.0) if init == "norm" else z * float(np.float32(0.02))
        out[a:a + len(i)] = v.to(torch.bfloat16).to(torch.float32)
    return out.reshape(tuple(shape))


class RandomWeights:
    """name -> tensor for a Qwen2-MoE configuration, each drawn when asked for (nothing is kept:
    a model of tens of gigabytes never exists as a whole).  Tensor names as in the checkpoints
    the reference reads (src/models/model.hip:487-512, 530-532, 559, 576, 586-587, 619) plus
    Qwen2-MoE's own (q/k/v biases, per-expert matrices, shared expert and its gate)."""

    def __init__(self, cfg: dict, seed: int, device="cpu"):
        self.seed, self.device = seed, device
        H, V = cfg["hidden_size"], cfg["vocab_size"]
        Hq = cfg["num_attention_heads"]
        Hkv = cfg.get("num_key_value_heads", Hq)
        D = cfg.get("head_dim") or H // Hq
        t = {"model.embed_tokens.weight": ((V, H), "linear"), "model.norm.weight": ((H,), "norm")}
        if not cfg.get("tie_word_embeddings"):
            t["lm_head.weight"] = ((V, H), "linear")
        for l in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{l}."
            t[p + "input_layernorm.weight"] = ((H,), "norm")
            t[p + "post_attention_layernorm.weight"] = ((H,), "norm")
            for n, rows in (("q", Hq * D), ("k", Hkv * D), ("v", Hkv * D)):
                t[p + f"self_attn.{n}_proj.weight"] = ((rows, H), "linear")
                if cfg.get("qkv_bias", True):
                    t[p + f"self_attn.{n}_proj.bias"] = ((rows,), "linear")
            t[p + "self_attn.o_proj.weight"] = ((H, Hq * D), "linear")
            if layer_is_sparse(cfg, l):
                I, Is = cfg["moe_intermediate_size"], cfg.get("shared_expert_intermediate_size", 0)
                t[p + "mlp.gate.weight"] = ((cfg["num_experts"], H), "linear")
                for e in range(cfg["num_experts"]):
                    q = f"{p}mlp.experts.{e}."
                    t[q + "gate_proj.weight"], t[q + "up_proj.weight"] = ((I, H), "linear"), ((I, H), "linear")
                    t[q + "down_proj.weight"] = ((H, I), "linear")
                if Is:
                    q = p + "mlp.shared_expert."
                    t[q + "gate_proj.weight"], t[q + "up_proj.weight"] = ((Is, H), "linear"), ((Is, H), "linear")
                    t[q + "down_proj.weight"] = ((H, Is), "linear")
                    t[p + "mlp.shared_expert_gate.weight"] = ((1, H), "linear")
            else:
                I = cfg["intermediate_size"]
                t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"] = ((I, H), "linear"), ((I, H), "linear")
                t[p + "mlp.down_proj.weight"] = ((H, I), "linear")
        self.tensors = t

    def __contains__(self, name):
        return name in self.tensors

    def __getitem__(self, name):
        shape, init = self.tensors[name]
        return plain_random_tensor(self.seed, name, shape, init, self.device)

    def keys(self):
        return self.tensors.keys()


# ---- parts ----------------------------------------------------------------------------

def plain_embedding(embed: torch.Tensor, tokens: List[int]) -> torch.Tensor:
    """h0[t] = embed[token[t]], no scaling (src/ops/kernels.hip:150-159)."""
    return embed[torch.tensor(tokens, dtype=torch.long, device=embed.device)]


def plain_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """inv = rsqrt(mean(x^2) + eps); y = x * inv * w; the weight multiplies directly
    (src/ops/kernels.hip:22-39)."""
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * inv * w


def plain_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq[i] = pow(theta, -2 i / D) in single precision
    (src/models/model.hip:636-639)."""
    out = []
    for i in range(head_dim // 2):
        expo = np.float32(np.float32(-2.0) * np.float32(i) / np.float32(head_dim))
        out.append(np.float32(math.pow(float(np.float32(theta)), float(expo))))
    return torch.tensor(np.array(out, dtype=np.float32))


def plain_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of [T, heads, D] (src/ops/kernels.hip:85-92):
    angle = float(pos) * inv_freq[i]; x'[i] = x[i] cos - x[i+D/2] sin;
    x'[i+D/2] = x[i] sin + x[i+D/2] cos.  The angle is formed in float32 as there."""
    half = x.shape[-1] // 2
    angle = (positions.to(torch.float32)[:, None] * inv_freq[None, :]).to(x.dtype)  # [T, D/2]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    window: Optional[int] = None) -> torch.Tensor:
    """q [T, Hq, D], k, v [T, Hkv, D] -> [T, Hq*D].  Query head h reads kv head
    h // (Hq/Hkv) (src/ops/attention.hip:27-28, 157-158); score = q.k / sqrt(D)
    (src/models/model.hip:285); key j visible to row t iff j <= t (attention.hip:216);
    softmax over the visible keys; o = sum p_j v_j (attention.hip:260-266).
    With a window w (not in the reference): visible iff t - w < j <= t."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    out = torch.zeros(T, Hq, D, dtype=q.dtype, device=q.device)
    idx = torch.arange(T, device=q.device)
    mask = idx[None, :] <= idx[:, None]
    if window:
        mask &= idx[None, :] > idx[:, None] - window
    for h in range(Hq):
        kh, vh = k[:, h // rep], v[:, h // rep]
        s = (q[:, h] @ kh.T) / math.sqrt(D)
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h] = p @ vh
    return out.reshape(T, Hq * D)


def plain_silu(z: torch.Tensor) -> torch.Tensor:
    """silu(z) = z / (1 + exp(-z)) (src/ops/kernels.hip:136-138)."""
    return z / (1.0 + torch.exp(-z))


def plain_swiglu_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                     w_down: torch.Tensor) -> torch.Tensor:
    """down(silu(gate x) * up x), no biases (src/models/model.hip:334-336)."""
    return (plain_silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def plain_router(x: torch.Tensor, w_router: torch.Tensor, k: int, norm_topk: bool,
                 forced_idx: Optional[torch.Tensor] = None):
    """Logits, softmax over all experts with the maximum subtracted, the k largest in
    descending order (src/ops/moe.hip:63-76; ties to the lower index here), weights
    p_e / sum(selected) when norm_topk (moe.hip:77-82, the only form the reference has)
    or p_e unchanged (Qwen2-MoE's norm_topk_prob=false).

    `forced_idx` [T, k] replaces the selection (not the probabilities): the comparison with
    a reduced-precision engine uses the engine's own choice, so that a near-tie decided the
    other way does not count as an error.  Returns (idx, weights, probabilities)."""
    logits = x @ w_router.T
    p = torch.softmax(logits, dim=-1)
    T, E = p.shape
    idx = torch.zeros(T, k, dtype=torch.long)
    wts = torch.zeros(T, k, dtype=x.dtype)
    p_host = p.cpu()
    for t in range(T):
        if forced_idx is not None:
            order = [int(e) for e in forced_idx[t]]
        else:
            order = sorted(range(E), key=lambda e: (-float(p_host[t, e]), e))[:k]
        idx[t] = torch.tensor(order)
        wts[t] = p_host[t, order]
    if norm_topk:
        wts = wts / wts.sum(dim=-1, keepdim=True)
    return idx.to(x.device), wts.to(x.device), p


def plain_sparse_ffn(x: torch.Tensor, weights, prefix: str, cfg: dict,
                     forced_idx: Optional[torch.Tensor] = None, slack: Optional[list] = None,
                     chosen: Optional[list] = None) -> torch.Tensor:
    """Routed experts summed in selection order with their routing weights
    (src/models/model.hip:355-433), plus the shared expert scaled by the sigmoid of its
    gate logit (Qwen2-MoE; absent from the reference).

    With `forced_idx`, `slack` (a list) receives for every row how far the forced choice
    falls short of the best one: (k-th largest probability - smallest forced probability)
    / k-th largest, 0 when the choice is the plain one.  `chosen` (a list) receives the experts
    used, [T, k]."""
    E, k = cfg["num_experts"], cfg["num_experts_per_tok"]
    idx, wts, prob = plain_router(x, weights[prefix + "gate.weight"], k,
                                  bool(cfg.get("norm_topk_prob", False)), forced_idx)
    if chosen is not None:
        chosen.append(idx.cpu())
    if forced_idx is not None and slack is not None:
        kth = torch.topk(prob, k, dim=-1).values[:, -1]
        worst = torch.gather(prob, 1, idx).min(dim=-1).values
        slack.append(((kth - worst) / kth).clamp_min(0))
    out = torch.zeros_like(x)
    # selection place by selection place, so that a row's sum runs in selection order; the
    # rows that chose the same expert at the same place share one pass over its matrices
    for j in range(k):
        for e in sorted(set(int(v) for v in idx[:, j])):
            rows = torch.nonzero(idx[:, j] == e).flatten()
            q = f"{prefix}experts.{e}."
            y = plain_swiglu_mlp(x[rows], weights[q + "gate_proj.weight"],
                                 weights[q + "up_proj.weight"], weights[q + "down_proj.weight"])
            out[rows] += wts[rows, j:j + 1] * y
    if cfg.get("shared_expert_intermediate_size", 0):
        q = prefix + "shared_expert."
        sh = plain_swiglu_mlp(x, weights[q + "gate_proj.weight"], weights[q + "up_proj.weight"],
                              weights[q + "down_proj.weight"])
        gamma = 1.0 / (1.0 + torch.exp(-(x @ weights[prefix + "shared_expert_gate.weight"].T)))
        out = out + gamma * sh
    return out


def layer_is_sparse(cfg: dict, l: int) -> bool:
    """Qwen2-MoE's rule; the reference treats every layer of an MoE model as sparse
    (src/models/model.hip:570)."""
    return (l not in (cfg.get("mlp_only_layers") or []) and cfg.get("num_experts", 0) > 0
            and (l + 1) % cfg.get("decoder_sparse_step", 1) == 0)


def layer_window(cfg: dict, l: int) -> Optional[int]:
    """The window of layer l, from config.json's own per-layer list; the reference has no
    window (src/ops/attention.hip:216 masks by `j <= p` alone)."""
    if cfg.get("use_sliding_window") and cfg["layer_types"][l] == "sliding_attention":
        return int(cfg["sliding_window"])
    return None


# ---- the whole model ------------------------------------------------------------------

class _As:
    """A name -> tensor mapping seen in another dtype, converted when asked for (the mapping
    may draw its tensors on demand, so nothing is touched before it is needed)."""

    def __init__(self, weights, dtype):
        self.weights, self.dtype = weights, dtype

    def __getitem__(self, name):
        return self.weights[name].to(self.dtype)

    def __contains__(self, name):
        return name in self.weights


def plain_forward(cfg: dict, weights, tokens: List[int], dtype: torch.dtype = torch.float32,
                  forced: Optional[Dict[int, torch.Tensor]] = None, slack: Optional[list] = None,
                  chosen: Optional[Dict[int, torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one request's whole token list.

    `forced` maps a sparse layer's index to the experts [T, k] its rows are to use (see
    `plain_router`); `slack` collects how far those choices are from the plain ones; `chosen`
    (a dictionary) receives the experts each sparse layer used.

    Layer order as src/models/model.hip:206-444: x1 = norm(h); qkv (+ bias, Qwen2-MoE);
    rotate q, k; attention; h += o_proj(attn); x2 = norm(h); ffn; h += ffn.  The
    reference adds the attention output to h a second time on its MoE branch
    (model.hip:311 and 440-444); that is a defect and is not restated.  Final norm and
    the head (tied to the embedding when tie_word_embeddings, model.hip:497-499,
    727-755)."""
    W = _As(weights, dtype)
    H = cfg["hidden_size"]
    Hq = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads", Hq)
    D = cfg.get("head_dim") or H // Hq
    eps = cfg.get("rms_norm_eps", 1e-6)
    T = len(tokens)
    h = plain_embedding(W["model.embed_tokens.weight"], tokens)
    inv_freq = plain_inv_freq(D, cfg.get("rope_theta", 1e6)).to(h.device)
    pos = torch.arange(T, device=h.device)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        x1 = plain_rms_norm(h, W[p + "input_layernorm.weight"], eps)
        q = x1 @ W[p + "self_attn.q_proj.weight"].T
        k = x1 @ W[p + "self_attn.k_proj.weight"].T
        v = x1 @ W[p + "self_attn.v_proj.weight"].T
        if p + "self_attn.q_proj.bias" in W:
            q = q + W[p + "self_attn.q_proj.bias"]
            k = k + W[p + "self_attn.k_proj.bias"]
            v = v + W[p + "self_attn.v_proj.bias"]
        q = plain_rope(q.reshape(T, Hq, D), pos, inv_freq)
        k = plain_rope(k.reshape(T, Hkv, D), pos, inv_freq)
        a = plain_attention(q, k, v.reshape(T, Hkv, D), layer_window(cfg, l))
        h = h + a @ W[p + "self_attn.o_proj.weight"].T
        x2 = plain_rms_norm(h, W[p + "post_attention_layernorm.weight"], eps)
        if layer_is_sparse(cfg, l):
            used = [] if chosen is not None else None
            f = plain_sparse_ffn(x2, W, p + "mlp.", cfg, None if forced is None else forced[l], slack, used)
            if chosen is not None:
                chosen[l] = used[0]
        else:
            f = plain_swiglu_mlp(x2, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                                 W[p + "mlp.down_proj.weight"])
        h = h + f
    n = plain_rms_norm(h, W["model.norm.weight"], eps)
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else W["lm_head.weight"]
    return n @ head.T


def plain_greedy(cfg: dict, weights: Dict[str, torch.Tensor], prompt: List[int], steps: int,
                 dtype: torch.dtype = torch.float32) -> List[int]:
    """Greedy generation by re-running the whole sequence each step: argmax, first maximum
    (src/runtime/engine.cpp:31-34)."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        logits = plain_forward(cfg, weights, ids, dtype)
        nxt = int(torch.argmax(logits[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out
