"""Plain, slow restatement of the Perelorn design in float64-free fp32 PyTorch: one function per mechanism, token by token,
no cache, no batching.  It shares no code with the product path (``mlx_sharding_b200``); the tests compare the framework to it.

Notation: ``h`` is the sublayer input ``[T, W]`` of ONE sequence whose first row is position 0; weights are a dict name -> fp32
tensor with the checkpoint names (``l<i>.mix.in`` ...).
"""
import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1 + torch.erf(z / math.sqrt(2)))


def silu(z):
    return z * torch.sigmoid(z)


def mamba2(h, w, p, m, eps):
    """State-space-duality mixer, sequential form."""
    T = h.shape[0]
    H, P, N, G, K, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner = H * P
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    cw, cb = w[p + "conv"], w[p + "conv.b"]
    pad = torch.cat([torch.zeros(K - 1, xbc.shape[1]), xbc])
    conv = torch.stack([(pad[t:t + K] * cw.T).sum(0) + cb for t in range(T)])
    conv = silu(conv)
    x, B, C = conv[:, :inner].view(T, H, P), conv[:, inner:inner + G * N].view(T, G, N), conv[:, inner + G * N:].view(T, G, N)
    dt = torch.logaddexp(torch.zeros(()), dt + w[p + "dt_bias"])
    A = -torch.exp(w[p + "A_log"])
    y = torch.zeros(T, H, P)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P)
        for t in range(T):
            S = torch.exp(A[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms(y.view(T, NG, inner // NG), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def rotate(v, pos, base, dims):
    """Rotate-half rotary on the first ``dims`` entries of the last axis; ``pos`` is [T]."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=torch.float32) / dims)
    a = pos.float()[:, None] * f
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = torch.cos(a).view(shape), torch.sin(a).view(shape)
    u1, u2 = v[..., :half], v[..., half:dims]
    return torch.cat([u1 * c - u2 * s, u2 * c + u1 * s, v[..., dims:]], -1)


def latent_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, D, R, V, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, D + R)
    kv = h @ w[p + "dkv"].T
    c = rms(kv[:, :L], eps) * w[p + "dkv.norm"]
    kr = rotate(kv[:, L:], pos, m["rot"]["base"], m["rot"]["dims"])
    qr = rotate(q[..., D:], pos, m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, V)
    out = torch.zeros(T, H, V)
    for hd in range(H):
        for t in range(T):
            s = (kn[:t + 1, hd] @ q[t, hd, :D] + kr[:t + 1] @ qr[t, hd]) * m["scale"]
            mx = torch.maximum(s.max(), w[p + "sink"][hd])
            e = torch.exp(s - mx)
            out[t, hd] = (e[:, None] * v[:t + 1, hd]).sum(0) / (e.sum() + torch.exp(w[p + "sink"][hd] - mx))
    return out.reshape(T, H * V) @ w[p + "o"].T


def lightning(h, w, p, m, eps):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q, k = silu(h @ w[p + "q"].T).view(T, H, D), silu(h @ w[p + "k"].T).view(T, H, D)
    v = silu(h @ w[p + "v"].T).view(T, H, V)
    o = torch.zeros(T, H, V)
    for hd in range(H):
        S = torch.zeros(D, V)
        for t in range(T):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms(o.reshape(T, H * V), eps) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


MIXERS = {"mamba2": mamba2, "latent_attention": latent_attention, "lightning": lightning}


def dense_ff(h, w, p):
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def side_input(x, tokens, w, i, dim, eps):
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ w[f"l{i}.side.gate"].T) * e) @ w[f"l{i}.side.proj"].T
    return x + rms(y, eps) * w[f"l{i}.side.norm"]


def forward(cfg, w, tokens, return_layers=False):
    """Logits ``[T, vocab]`` of one whole sequence (and the residual stream after every layer)."""
    w = {k: v.float() for k, v in w.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = w["embed"][tokens]
    layers = []
    for i, L in enumerate(cfg["layers"]):
        x = x + rms(MIXERS[L["type"]](x, w, f"l{i}.mix.", L["mixer"], eps), eps) * w[f"l{i}.norm1"]
        if L.get("mlp"):
            x = x + rms(dense_ff(x, w, f"l{i}.mlp."), eps) * w[f"l{i}.norm2"]
        if cfg.get("token_side"):
            x = side_input(x, tokens, w, i, cfg["token_side"]["dim"], eps)
        layers.append(x)
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(layers)) if return_layers else logits
