"""A plain, slow restatement of the Ganidra design, one function per mechanism.

Everything runs on the CPU in one floating-point type (float64 by default), token
by token where the design is recurrent, with no cache, no batching and no code
of the package.  The tests compare the engine with it.

Notation: ``x`` [T, W] is the residual stream of ONE sequence, positions 0..T-1;
``w`` maps tensor names to tensors; ``cfg`` is the parsed config.json.
"""
from __future__ import annotations

import math

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, weight, eps):
    """The layer norm of the design: the stored weight sits around zero."""
    return rms_unit(x, eps) * (1.0 + weight)


def norm_plain(x, weight, eps):
    return rms_unit(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def embed_tokens(tokens, table, scale):
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


def channel_decay(h, w_a1, w_a2, bias, tau):
    """alpha [T, heads*dim] in (0, 1): sigmoid(z) ** (1 / tau), z from the low-rank pair."""
    z = (h @ w_a1.T) @ w_a2.T + bias
    return torch.sigmoid(z) ** (1.0 / tau)


def linear_attention_recurrence(q, k, v, alpha):
    """One head, token by token.  q, k, alpha [T, dk]; v [T, dv].  S starts at zero;
    S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t."""
    T, dk = q.shape
    dv = v.shape[1]
    S = torch.zeros(dk, dv, dtype=q.dtype)
    out = torch.zeros(T, dv, dtype=q.dtype)
    for t in range(T):
        S = alpha[t][:, None] * S + k[t][:, None] * v[t][None, :]
        out[t] = S.T @ q[t]
    return out


def gla_mixer(h, w, p, m, eps):
    """The gated-linear-attention mixer.  ``p`` is the tensor prefix ('l0.mix.'), ``m`` its sizes."""
    T = h.shape[0]
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ w[p + "q"].T) * dk ** -0.5
    k = h @ w[p + "k"].T
    v = h @ w[p + "v"].T
    alpha = channel_decay(h, w[p + "a1"], w[p + "a2"], w[p + "a2.b"], tau)
    heads = []
    for i in range(H):
        o = linear_attention_recurrence(q[:, i * dk:(i + 1) * dk], k[:, i * dk:(i + 1) * dk],
                                        v[:, i * dv:(i + 1) * dv], alpha[:, i * dk:(i + 1) * dk])
        heads.append(norm_plain(o, w[p + "norm"], eps))
    o = torch.cat(heads, dim=1) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def distance_slopes(num_heads):
    return [2.0 ** (-8.0 * (i + 1) / num_heads) for i in range(num_heads)]


def windowed_softmax_attention(q, k, v, scale, slope, window):
    """One head.  q, k [T, dk]; v [T, dv].  The query at i sees j with 0 <= i - j < window; the score
    is scale * q.k - slope * (i - j); plain softmax over what is seen."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=q.dtype)
    for i in range(T):
        lo = max(0, i - window + 1)
        js = torch.arange(lo, i + 1)
        s = (k[lo:i + 1] @ q[i]) * scale - slope * (i - js).to(q.dtype)
        p = torch.softmax(s, dim=0)
        out[i] = p @ v[lo:i + 1]
    return out


def softmax_mixer(h, w, p, m, eps):
    """The softmax mixer of the parallel layer: grouped heads, q/k norm, distance bias, window, output gate."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[p + "q"].T
    k = h @ w[p + "k"].T
    v = h @ w[p + "v"].T
    slopes = distance_slopes(H)
    heads = []
    for i in range(H):
        g = i // (H // G)
        qi = norm_plain(q[:, i * dk:(i + 1) * dk], w[p + "q.norm"], eps)
        ki = norm_plain(k[:, g * dk:(g + 1) * dk], w[p + "k.norm"], eps)
        heads.append(windowed_softmax_attention(qi, ki, v[:, g * dv:(g + 1) * dv], m["scale"], slopes[i],
                                                m["mask"]["size"]))
    o = torch.cat(heads, dim=1) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    left = softmax_mixer(h, w, p + "left.", m["left"], eps)
    right = gla_mixer(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def mixer(kind, h, w, p, m, eps):
    if kind == "gla":
        return gla_mixer(h, w, p, m, eps)
    if kind == "parallel":
        return parallel_mixer(h, w, p, m, eps)
    raise ValueError(kind)


def gated_feed_forward(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def layer(x, w, i, spec, eps):
    p = f"l{i}."
    x = x + mixer(spec["type"], norm_one_plus(x, w[p + "norm1"], eps), w, p + "mix.", spec["mixer"], eps)
    if spec.get("mlp") is not None:
        x = x + gated_feed_forward(norm_one_plus(x, w[p + "norm2"], eps), w, p + "mlp.")
    return x


def layer_order(cfg):
    """[(layer index, embedding added before it)] in the order of running."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    if b <= a or times <= 1:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(a)]
    for t in range(times):
        order += [(i, t > 0 and i == a) for i in range(a, b)]
    order += [(i, False) for i in range(b, n)]
    return order


def forward(cfg, w, tokens, dtype=torch.float64, keep_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer run)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    e = embed_tokens(tokens, w["embed"], cfg["embedding"]["scale"])
    x = e
    kept = []
    for i, again in layer_order(cfg):
        if again:
            x = x + e
        x = layer(x, w, i, cfg["layers"][i], eps)
        if keep_layers:
            kept.append(x.clone())
    logits = norm_one_plus(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, kept) if keep_layers else logits


def read_model_folder(folder: str):
    """(config.json as a dict, {tensor name: tensor}) of a model folder."""
    import json
    import os

    from safetensors import safe_open
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            w[name] = f.get_tensor(name)
    return cfg, w


def greedy(cfg, w, prompt, n_new, dtype=torch.float64):
    """The prompt's greedy continuation, token by token over the whole sequence each time."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(cfg, w, toks, dtype)[-1])))
    return toks[len(prompt):]
