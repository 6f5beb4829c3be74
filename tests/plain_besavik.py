"""Besavik, written down plainly: one function per mechanism, float64, token by
token where the design is a recurrence, no cache, no batch, no code of the
package.  The tests compare the engine with this.

Notation: h is a mixer's input [T, W] (the normed stream), weights are a dict
name -> tensor stored [out, in] and applied as W h.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotate_half_pairs(x, positions, base, dims):
    """x [T, ..., D]: the first ``dims`` channels are rotated, channel i with channel i + dims/2, by the
    angle position * base^(-2i/dims); the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(F64)[:, None] * freq[None, :]                 # [T, half]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def latent_softmax(q_plain, q_rot, k_plain, k_rot, v, scale, first=0):
    """Causal softmax attention with a key part that all heads share.  q_plain [n, H, dn], q_rot [n, H, dr] (already
    rotated) are the queries at positions first .. first + n - 1; k_plain [t, H, dn], k_rot [t, dr], v [t, H, dv]
    the keys and values of positions 0 .. t - 1."""
    n, H = q_plain.shape[:2]
    out = torch.zeros(n, H, v.shape[-1], dtype=F64)
    for i in range(n):
        last = first + i + 1
        s = (torch.einsum("hd,jhd->hj", q_plain[i], k_plain[:last]) + torch.einsum("hd,jd->hj", q_rot[i], k_rot[:last])) * scale
        out[i] = torch.einsum("hj,jhd->hd", torch.softmax(s, dim=-1), v[:last])
    return out


def latent_attention(h, w, p, m, eps, positions=None):
    """Softmax attention whose keys and values are read out of a small latent per token, with one rotated key
    part shared by all heads.  m: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {base, dims}."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], q[..., dn:]
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :r], w[p + "dkv.norm"], eps)
    k_rot = down[:, r:]                                               # [T, dr], one for all heads
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q_rot = rotate_half_pairs(q_rot, pos, base, dims)
    k_rot = rotate_half_pairs(k_rot, pos, base, dims)
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    out = latent_softmax(q_plain, q_rot, k_plain, k_rot, v, m["scale"])
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T


def decayed_recurrence(q, k, v, decay, S=None):
    """S <- decay_h S + k v^T, o = S^T q per head; q, k [T, H, dk], v [T, H, dv], decay [H].  Returns o and the last S."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=F64) if S is None else S
    o = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def lightning(h, w, p, m, eps):
    """Linear attention with one constant decay per head: S <- decay S + k v^T, o = S^T q."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ w[p + "q"].T).reshape(T, H, dk)
    k = silu(h @ w[p + "k"].T).reshape(T, H, dk)
    v = silu(h @ w[p + "v"].T).reshape(T, H, dv)
    o, _ = decayed_recurrence(q, k, v, torch.tensor(m["decay"], dtype=F64))
    y = rms_norm(o.reshape(T, H * dv), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def short_conv(x, taps_w):
    """x [T, C]; taps_w [C, taps]: tap taps - 1 multiplies the token itself, and inputs before the first token count as zero."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j][None, :]
    return y


def delta_recurrence(q, k, v, g, beta, S=None):
    """S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q per head, in this order.  q, k, g [T, H, dk]
    (q and k already repeated for the heads of a group), v [T, H, dv], beta [T, H].  Returns o and the last S."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=F64) if S is None else S
    o = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def channel_delta(h, w, p, m, eps):
    """The gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                           # [T, H]
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    rate = torch.exp(w[p + "A_log"])                                 # [H]
    g = torch.exp(-rate[None, :, None] * torch.nn.functional.softplus(z).reshape(T, H, dk))
    rep = H // G                                                      # head h reads q/k head h // rep
    o, _ = delta_recurrence(q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1), v, g, beta)
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * w[p + "norm"]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T)
    return (o.reshape(T, H * dv) * gate) @ w[p + "o"].T


def limited_glu(h, w_gate, w_up, w_down, limit):
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def dense_ff(h, w, p, mlp):
    return limited_glu(h, w[p + "gate"], w[p + "up"], w[p + "down"], mlp["limit"])


def route(h, w_router, bias, top):
    """The experts a token uses and their weights: the `top` largest logits, softmax over those alone."""
    z = h @ w_router.T + bias
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe_ff(h, w, p, mlp):
    top = mlp["router"]["top"]
    idx, wgt = route(h, w[p + "router"], w[p + "router.b"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            pe = f"{p}e{e}."
            out[t] += wgt[t, j] * limited_glu(h[t:t + 1], w[pe + "gate"], w[pe + "up"], w[pe + "down"],
                                              mlp["expert"]["limit"])[0]
    return out


MIXERS = {"latent_attention": latent_attention, "lightning": lightning, "channel_delta": channel_delta}


def forward(cfg: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = rms_norm(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], w["embed.norm"], eps)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        x = x + MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            x = x + (dense_ff if mlp["kind"] == "dense" else moe_ff)(h, w, p + "mlp.", mlp)
        after.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T * cfg["logit_scale"]
    return (logits, torch.stack(after)) if return_layers else logits


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


def greedy(cfg, w, prompt, n_new):
    """The prompt's greedy continuation, token by token over the whole sequence each time."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]
