"""Plain, slow implementation of the Llama / Qwen2 dense decoder.

This file rests on the formulas of yudono/rust-inference's CPU code: the crate is a
binary with private modules that needs a Rust toolchain and crates from the network,
neither of which exists here, so it cannot be imported or compiled for a golden run.
Every function below cites the lines of the reference that it restates.  In place of a
golden run of the reference, `tests/golden/` holds a second, independent statement of the
same formulas (a scalar C++ program: loops, one token at a time, a cache), the logits it
computes on two tiny models, and the script that made them; `tests/test_plain_impl.py`
compares this file with them.

It processes whole sequences, keeps no cache, has one function for each part and
shares no code with the package under test: it only uses torch tensor arithmetic
on the CPU (or wherever its inputs live), in float32 unless told otherwise.

Weights are passed as a dict from safetensors tensor name to tensor, the
configuration as the plain dict read from config.json.
"""
from __future__ import annotations

import math

import torch


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def embedding(table: torch.Tensor, ids) -> torch.Tensor:
    """h = token_embd[token_id, :]   (transformer.rs:74-75, quant.rs:152-174)."""
    idx = torch.as_tensor(ids, dtype=torch.long, device=table.device)
    return table[idx]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum x^2; rms = sqrt(ss/n + eps); y = x * (1/rms) * w   (math.rs:237-256,
    rmsnorm.rs:18-29).  eps sits inside the square root, added to the mean."""
    n = x.shape[-1]
    ss = (x * x).sum(dim=-1, keepdim=True)
    rms = torch.sqrt(ss / n + eps)
    scale = 1.0 / rms
    return x * scale * weight


def rope_table(head_dim: int, base: float, n_pos: int, dtype=torch.float32):
    """cos/sin tables [n_pos, head_dim/2]   (rope.rs:42-64).

    exponent = 2i/dim, theta = 1/base^exponent, angle = pos*theta; theta and the
    angle are 32-bit numbers in the reference, so they are rounded to float32 here
    (the power itself is taken in float64 and rounded once, which is what a
    correctly rounded powf returns).  cos and sin are taken of that 32-bit angle."""
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    exponent = ((2 * i).to(torch.float32) / torch.tensor(float(head_dim), dtype=torch.float32))
    theta = (1.0 / torch.pow(torch.tensor(float(base), dtype=torch.float32).double(),
                             exponent.double())).to(torch.float32)
    pos = torch.arange(n_pos, dtype=torch.float32)
    angle = (pos[:, None] * theta[None, :]).to(torch.float32)   # f32 product
    cos = torch.cos(angle.double()).to(torch.float32)
    sin = torch.sin(angle.double()).to(torch.float32)
    return cos.to(dtype), sin.to(dtype)


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, style: str) -> torch.Tensor:
    """Rotate one head's vectors.  x: [n, head_dim]; cos, sin: [n, head_dim/2].

    style "interleaved": pairs (2i, 2i+1)   (rope.rs:88-97):
        x'[2i] = x[2i] c - x[2i+1] s ;  x'[2i+1] = x[2i] s + x[2i+1] c
    style "half": pairs (i, i + dim/2), the pairing that safetensors checkpoints of
    this architecture are laid out for; same angles."""
    out = torch.empty_like(x)
    half = x.shape[-1] // 2
    if style == "interleaved":
        x0, x1 = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = x0 * cos - x1 * sin
        out[..., 1::2] = x0 * sin + x1 * cos
    elif style == "half":
        x0, x1 = x[..., :half], x[..., half:]
        out[..., :half] = x0 * cos - x1 * sin
        out[..., half:] = x0 * sin + x1 * cos
    else:
        raise ValueError(style)
    return out


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """y_r = sum_c W[r, c] x_c (+ b_r); weights are [out, in], row-major over `in`
    (quant.rs:178-206, math.rs:212-229)."""
    y = x @ w.t()
    if b is not None:
        y = y + b
    return y


def softmax_rows(s: torch.Tensor) -> torch.Tensor:
    """m = max; e = exp(s - m); p = e * (1/sum e)   (math.rs:104-118)."""
    m = s.max(dim=-1, keepdim=True).values
    e = torch.exp(s - m)
    return e * (1.0 / e.sum(dim=-1, keepdim=True))


def stored(x: torch.Tensor, store_dtype) -> torch.Tensor:
    """x as it reads back after being kept in `store_dtype` (None: unchanged).  The arithmetic of
    this file is float32 throughout, as the reference's is; this only restates what keeping
    activations and the cache in bfloat16 between two operations does to the numbers, so that a
    test can tell how much of a bfloat16 run's distance from float32 is storage rounding."""
    return x if store_dtype is None else x.to(store_dtype).to(x.dtype)


def attention(x: torch.Tensor, p: dict, prefix: str, *, n_heads: int, n_kv_heads: int,
              head_dim: int, cos: torch.Tensor, sin: torch.Tensor, rope_style: str,
              window: int | None = None, kv_from: tuple | None = None, store_dtype=None):
    """Grouped-query attention over one whole sequence (attention.rs:54-124).

    q = Wq x + bq, k = Wk x + bk, v = Wv x + bv (:66-76); rope on every q head and
    every k head at the token's position (:78-87); query head h uses kv head
    h / n_rep with n_rep = n_heads / n_kv_heads (:37, :95-98); scores = dot * scale,
    scale = 1/sqrt(head_dim) applied to the finished dot product (:100-110); the
    token at position t sees keys 0..t only (causal by construction, :92); softmax
    (:112); weighted sum of values (:114-120); output projection without bias (:123).

    `window` (not in the reference) restricts a query at t to keys t-window+1..t;
    `kv_from` lets the layer use keys and values another layer produced.  Returns
    (output, (k, v)) so that a later layer can be handed this layer's keys and values."""
    n = x.shape[0]
    q = linear(x, p[prefix + "q_proj.weight"], p.get(prefix + "q_proj.bias"))
    q = q.view(n, n_heads, head_dim)
    if kv_from is None:
        k = linear(x, p[prefix + "k_proj.weight"], p.get(prefix + "k_proj.bias"))
        v = linear(x, p[prefix + "v_proj.weight"], p.get(prefix + "v_proj.bias"))
        k = k.view(n, n_kv_heads, head_dim)
        v = v.view(n, n_kv_heads, head_dim)
        k = torch.stack([rope_apply(k[:, h], cos[:n], sin[:n], rope_style)
                         for h in range(n_kv_heads)], dim=1)
        k, v = stored(k, store_dtype), stored(v, store_dtype)          # the cache
    else:
        k, v = kv_from
    q = torch.stack([rope_apply(q[:, h], cos[:n], sin[:n], rope_style)
                     for h in range(n_heads)], dim=1)
    q = stored(q, store_dtype)
    n_rep = n_heads // n_kv_heads
    scale = 1.0 / math.sqrt(float(head_dim))
    out = torch.zeros(n, n_heads, head_dim, dtype=x.dtype, device=x.device)
    pos = torch.arange(n, device=x.device)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible = visible & (pos[None, :] > pos[:, None] - window)
    for h in range(n_heads):
        kvh = h // n_rep
        s = (q[:, h] @ k[:, kvh].t()) * scale
        s = s.masked_fill(~visible, float("-inf"))
        out[:, h] = stored(softmax_rows(s), store_dtype) @ v[:, kvh]
    out = stored(out, store_dtype)
    y = linear(out.reshape(n, n_heads * head_dim), p[prefix + "o_proj.weight"])
    return y, (k, v)


def silu(x: torch.Tensor) -> torch.Tensor:
    """x/(1+exp(-x)) for x >= 0, x*exp(x)/(1+exp(x)) for x < 0   (math.rs:137-146)."""
    pos = x / (1.0 + torch.exp(-x.clamp(min=0)))
    e = torch.exp(x.clamp(max=0))
    neg = x * e / (1.0 + e)
    return torch.where(x >= 0, pos, neg)


def swiglu(x: torch.Tensor, p: dict, prefix: str, store_dtype=None) -> torch.Tensor:
    """down( silu(gate x) * (up x) ), no biases   (mlp.rs:31-46)."""
    g = silu(linear(x, p[prefix + "gate_proj.weight"]))
    u = linear(x, p[prefix + "up_proj.weight"])
    return linear(stored(g * u, store_dtype), p[prefix + "down_proj.weight"])


def block(x: torch.Tensor, p: dict, layer: int, cfg: dict, cos, sin, kv_from=None, store_dtype=None):
    """x + attn(norm(x)), then + mlp(norm(.))   (transformer.rs:20-48).  The residual stream stays
    float32 whatever `store_dtype` is."""
    pre = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    xn = stored(rmsnorm(x, p[pre + "input_layernorm.weight"], eps), store_dtype)
    a, kv = attention(xn, p, pre + "self_attn.", n_heads=cfg["num_attention_heads"],
                      n_kv_heads=cfg["num_key_value_heads"], head_dim=cfg["head_dim"],
                      cos=cos, sin=sin, rope_style=cfg.get("rope_style", "half"),
                      kv_from=kv_from, store_dtype=store_dtype)
    h1 = x + a
    xn2 = stored(rmsnorm(h1, p[pre + "post_attention_layernorm.weight"], eps), store_dtype)
    return h1 + swiglu(xn2, p, pre + "mlp.", store_dtype), kv


# ----------------------------------------------------------------------------
# whole model
# ----------------------------------------------------------------------------

def resolve_config(cfg: dict) -> dict:
    """The soft defaults the reference applies (model.rs:97-104, :86): kv heads = heads,
    head_dim = hidden/heads (model.rs:153), eps 1e-5; rope base by architecture."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    c.setdefault("rms_norm_eps", 1e-5)
    arch = c["architectures"][0]
    c.setdefault("rope_theta", 1e6 if arch.startswith("Qwen2") else 1e4)
    c.setdefault("tie_word_embeddings", False)
    return c


def row_stats(row: torch.Tensor) -> dict:
    """min, max, mean and the first four values of one hidden vector, as the reference's debug
    probe prints them for position 0 (transformer.rs:80-86, :90-96)."""
    return {"min": float(row.min()), "max": float(row.max()), "mean": float(row.sum() / row.numel()),
            "first": [float(v) for v in row[:4]]}


def forward(weights: dict, cfg: dict, tokens, schedule=None, dtype=torch.float32, stats=None,
            stats_position: int = 0, store_dtype=None) -> torch.Tensor:
    """Logits [n, vocab] at every position of one sequence (transformer.rs:63-98):
    embedding row, the layers in order, final RMSNorm, lm_head (the embedding matrix
    when tied, model.rs:221-226).

    `schedule` is the list of layers to run, as (weights_layer, reads_cache_of) pairs;
    the default is each layer once, in order, with its own keys and values.
    `stats`: a list that receives (label, row_stats) of the hidden vector at `stats_position`
    after every layer ("L0", "L1", ...) and after the final norm ("FNL").
    `store_dtype`: keep what passes from one operation to the next (normalised input, rotated q and
    k, v, probabilities, attention output, gated activation) in this dtype, see `stored`."""
    c = resolve_config(cfg)
    p = {k: v.to(dtype) for k, v in weights.items()}
    n = len(tokens)
    cos, sin = rope_table(c["head_dim"], c["rope_theta"], n, dtype=dtype)
    dev = p["model.embed_tokens.weight"].device
    cos, sin = cos.to(dev), sin.to(dev)
    h = embedding(p["model.embed_tokens.weight"], tokens)
    if schedule is None:
        schedule = [(i, None) for i in range(c["num_hidden_layers"])]
    produced = {}
    for run_idx, (layer, reads) in enumerate(schedule):
        kv_from = produced[reads] if reads is not None else None
        h, kv = block(h, p, layer, c, cos, sin, kv_from=kv_from, store_dtype=store_dtype)
        produced[run_idx] = kv
        if stats is not None:
            stats.append((f"L{run_idx}", row_stats(h[stats_position])))
    h = stored(rmsnorm(h, p["model.norm.weight"], c["rms_norm_eps"]), store_dtype)
    if stats is not None:
        stats.append(("FNL", row_stats(h[stats_position])))
    head = p["model.embed_tokens.weight"] if c["tie_word_embeddings"] else p["lm_head.weight"]
    return linear(h, head)


# ----------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------

def argmax_first(logits: torch.Tensor) -> int:
    """Index of the maximum, the first one on ties (strict >)   (math.rs:328-339)."""
    best, idx = logits[0].item(), 0
    vals = logits.tolist()
    for i in range(1, len(vals)):
        if vals[i] > best:
            best, idx = vals[i], i
    return idx


def repetition_penalty(logits: torch.Tensor, recent, penalty: float, window: int) -> torch.Tensor:
    """For each id among the last `window` of `recent` (repeats apply again):
    l > 0 ? l / p : l * p   (sampler.rs:109-127)."""
    out = logits.clone()
    start = max(0, len(recent) - window)
    for t in list(recent)[start:]:
        if t < out.numel():
            out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out


def top_k_filter(probs: torch.Tensor, k: int) -> torch.Tensor:
    """Zero everything below the k-th largest probability (ties kept), renormalise
    (sampler.rs:130-160)."""
    if k <= 0 or k >= probs.numel():
        return probs
    threshold = torch.sort(probs, descending=True).values[k - 1]
    out = torch.where(probs < threshold, torch.zeros_like(probs), probs)
    s = out.sum()
    return out * (1.0 / s) if s > 0 else out


def top_p_filter(probs: torch.Tensor, p: float) -> torch.Tensor:
    """Keep the smallest prefix of the descending (stable) order whose sum reaches p,
    zero the rest, renormalise   (sampler.rs:163-196)."""
    if not (0.0 < p < 1.0):
        return probs
    order = torch.sort(probs, descending=True, stable=True).indices
    csum = torch.cumsum(probs[order], dim=0)
    reached = (csum >= p).nonzero()
    cutoff = int(reached[0]) + 1 if reached.numel() else probs.numel()
    out = torch.zeros_like(probs)
    out[order[:cutoff]] = probs[order[:cutoff]]
    s = out.sum()
    return out * (1.0 / s) if s > 0 else out


def draw(probs: torch.Tensor, r: float) -> int:
    """First i whose running sum reaches r, else the last index   (sampler.rs:199-210)."""
    csum = torch.cumsum(probs, dim=0)
    hit = (csum >= r).nonzero()
    return int(hit[0]) if hit.numel() else probs.numel() - 1


def sample(logits: torch.Tensor, *, temperature: float, r: float, top_k: int = 0,
           top_p: float = 1.0, penalty: float = 1.0, window: int = 64, recent=()) -> int:
    """The reference's order of operations (sampler.rs:72-106): penalty, greedy if
    temperature <= 0, divide by temperature, softmax, top-k, top-p, draw with the
    uniform number r."""
    l = logits.clone().float()
    if penalty != 1.0 and len(recent):
        l = repetition_penalty(l, recent, penalty, window)
    if temperature <= 0.0:
        return argmax_first(l)
    probs = softmax_rows(l / temperature)
    probs = top_k_filter(probs, top_k)
    probs = top_p_filter(probs, top_p)
    return draw(probs, r)


def greedy_generate(weights: dict, cfg: dict, prompt, max_tokens: int, stop_ids=()) -> list:
    """Prefill, then sample / stop-check / forward (model.rs:361-442) with greedy
    sampling and no penalty; a sampled stop id ends the sequence and is not emitted
    (model.rs:383-387).  Recomputes the whole sequence for every token."""
    seq = list(prompt)
    out = []
    for _ in range(max_tokens):
        logits = forward(weights, cfg, seq)[-1]
        nxt = argmax_first(logits)
        if nxt in stop_ids:
            break
        out.append(nxt)
        seq.append(nxt)
    return out
