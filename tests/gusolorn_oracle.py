"""Plain, slow restatement of the Gusolorn design, one function per mechanism, straight from its equations.  It shares no code with
the package: dense tensors, whole sequences, Python loops over tokens; ``float64`` by default so that it can serve as ground truth.

A model is ``(cfg, sd)``: ``cfg`` the parsed ``config.json`` (keys ``layers``, ``norm.eps``, ``vocab``, ``width``), ``sd`` a dict
name -> tensor.  ``random_model(cfg, seed)`` draws weights for any configuration."""
import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotate_pairs(v, pos, base, dims):
    """``v`` [T, ..., dims]; adjacent pairs (2i, 2i+1) turn by ``pos * base^(-2i/dims)``."""
    out = v.clone()
    for i in range(dims // 2):
        a = pos.to(v.dtype) * (base ** (-2.0 * i / dims))
        while a.dim() < v.dim() - 1:
            a = a.unsqueeze(-1)
        c, s = torch.cos(a), torch.sin(a)
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def mlstm_mixer(h, p, m, eps):
    """``h`` [T, width] of one sequence from its start.  ``p``: tensors of the mixer (q k v g o norm i i.b f f.b)."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ p["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ p["k"].T).view(T, H, D)
    v = (h @ p["v"].T).view(T, H, V)
    ig = cap * torch.tanh((h @ p["i"].T + p["i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ p["f"].T + p["f.b"]) / cap))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        n = torch.zeros(D, dtype=h.dtype)
        mm = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            m_new = torch.maximum(fg[t, hd] + mm, ig[t, hd])
            a, b = torch.exp(fg[t, hd] + mm - m_new), torch.exp(ig[t, hd] - m_new)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mm = m_new
            den = torch.maximum(torch.abs(n @ q[t, hd]), torch.exp(-mm)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
    o = rms(out, eps).reshape(T, H * V) * p["norm"] * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


def latent_kv(h, p, m, eps):
    """What a latent-attention layer with its own down-projection caches: latent ``c`` [T, kv_rank], rotated shared key [T, rot_dim]."""
    T = h.shape[0]
    L, R = m["kv_rank"], m["rot_dim"]
    d = h @ p["dkv"].T
    c = rms(d[:, :L], eps) * p["dkv.norm"]
    kr = rotate_pairs(d[:, L:L + R], torch.arange(T), float(m["rot"]["base"]), int(m["rot"]["dims"]))
    return c, kr


def latent_attention_mixer(h, p, m, eps, shared_kv=None):
    """``shared_kv``: ``(c, kr)`` of the layer named by ``kv_from`` (then this layer has no down-projection)."""
    T = h.shape[0]
    H, D, R, V, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = shared_kv if shared_kv is not None else latent_kv(h, p, m, eps)
    q = (h @ p["q"].T).view(T, H, D + R)
    qn = q[..., :D]
    qr = rotate_pairs(q[..., D:], torch.arange(T), float(m["rot"]["base"]), int(m["rot"]["dims"]))
    kn = (c @ p["uk"].T).view(T, H, D)
    vv = (c @ p["uv"].T).view(T, H, V)
    win = int(m["mask"]["size"]) if m.get("mask") else None
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        lo = 0 if win is None else max(0, t - win + 1)
        for hd in range(H):
            s = (kn[lo:t + 1, hd] @ qn[t, hd] + kr[lo:t + 1] @ qr[t, hd]) * float(m["scale"])
            out[t, hd] = torch.softmax(s, 0) @ vv[lo:t + 1, hd]
    return out.reshape(T, H * V) @ p["o"].T, (c, kr)


def clamped_expert(x, p, limit):
    g = torch.clamp(x @ p["gate"].T, max=limit)
    u = torch.clamp(x @ p["up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ p["down"].T


ROUTER_GAPS = []       # per router call: smallest distance, over its tokens, between the last chosen logit and the first one left out


def router(h, w, top):
    """Scores ``sigmoid(W h)``; the ``top`` largest, weights = their scores as they are."""
    z = h @ w.T
    if top < z.shape[-1]:
        zs = torch.sort(z, dim=-1, descending=True).values
        ROUTER_GAPS.append(float((zs[:, top - 1] - zs[:, top]).min()))
    s = torch.sigmoid(z)
    wts, idx = torch.topk(s, top, dim=-1)
    return idx, wts


def feed_forward(h, p, mlp):
    if mlp["kind"] == "dense":
        return gelu_erf(h @ p["up"].T) @ p["down"].T
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, wts = router(h, p["router"], top)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            ep = {n: p[f"e{e}.{n}"] for n in ("gate", "up", "down")}
            y[t] += clamped_expert(wts[t, j] * h[t], ep, float(mlp["expert"]["limit"]))
    if mlp.get("shared"):
        sp = {n: p[f"shared.{n}"] for n in ("gate", "up", "down")}
        y = y + clamped_expert(h, sp, float(mlp["shared"]["limit"])) * torch.sigmoid(h @ p["shared.sg"].T)
    return y


def sub(sd, prefix):
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


def forward(cfg, sd, tokens, dtype=torch.float64, layers_out=None):
    """Logits ``[T, vocab]`` of one whole sequence."""
    sd = {k: v.to(dtype) for k, v in sd.items()}
    eps = float(cfg["norm"]["eps"])
    x = sd["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kv = {}
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = zero_centred_norm(x, sd[pre + "norm1"], eps)
        m = L["mixer"]
        if L["type"] == "mlstm":
            y = mlstm_mixer(h, sub(sd, pre + "mix."), m, eps)
        else:
            src = m.get("kv_from")
            y, kv[i] = latent_attention_mixer(h, sub(sd, pre + "mix."), m, eps, kv[src] if src is not None else None)
        x = x + y * sd[pre + "ls1"]
        if L.get("mlp"):
            h = zero_centred_norm(x, sd[pre + "norm2"], eps)
            x = x + feed_forward(h, sub(sd, pre + "mlp."), L["mlp"]) * sd[pre + "ls2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return zero_centred_norm(x, sd["final.norm"], eps) @ sd["head"].T


def min_router_gap(cfg, sd, tokens):
    """How far the sequence's routing is from a close call (logit units; inf without routing decisions)."""
    del ROUTER_GAPS[:]
    forward(cfg, sd, tokens)
    return min(ROUTER_GAPS, default=float("inf"))


def tensor_shapes(cfg):
    W, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],), "head": (cfg["vocab"], cfg["width"])}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"], out[p + "ls1"] = (W,), (W,)
        if L["type"] == "mlstm":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * D, W), p + "mix.k": (H * D, W), p + "mix.v": (H * V, W), p + "mix.g": (H * V, W), p + "mix.o": (W, H * V),
                        p + "mix.norm": (H * V,), p + "mix.i": (H, W), p + "mix.i.b": (H,), p + "mix.f": (H, W), p + "mix.f.b": (H,)})
        else:
            H, D, R, V, Lr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({p + "mix.q": (H * (D + R), W), p + "mix.uk": (H * D, Lr), p + "mix.uv": (H * V, Lr), p + "mix.o": (W, H * V)})
            if m.get("kv_from") is None:
                out.update({p + "mix.dkv": (Lr + R, W), p + "mix.dkv.norm": (Lr,)})
        mlp = L.get("mlp")
        if mlp:
            out[p + "norm2"], out[p + "ls2"] = (W,), (W,)
            if mlp["kind"] == "dense":
                out.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                F = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    out.update({p + f"mlp.e{e}.gate": (F, W), p + f"mlp.e{e}.up": (F, W), p + f"mlp.e{e}.down": (W, F)})
                out[p + "mlp.router"] = (mlp["router"]["experts"], W)
                if mlp.get("shared"):
                    Fs = mlp["shared"]["ff"]
                    out.update({p + "mlp.shared.gate": (Fs, W), p + "mlp.shared.up": (Fs, W), p + "mlp.shared.down": (W, Fs), p + "mlp.shared.sg": (1, W)})
    return out


def random_model(cfg, seed=0, dtype=torch.bfloat16):
    """Random weights on the bf16 grid: projections ~ N(0, 1/fan_in) (gate rows larger so the caps and the running maximum are
    exercised), norm weights and layer scales around 0 / 1, router rows large enough that choices are not close calls."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if len(shape) == 1:
            if leaf in ("ls1", "ls2"):
                t = 1.0 + 0.2 * torch.randn(shape, generator=g)
            elif name.endswith("mix.norm") or name.endswith("dkv.norm"):
                t = 1.0 + 0.1 * torch.randn(shape, generator=g)
            elif leaf == "b":
                t = 2.0 * torch.randn(shape, generator=g) + (3.0 if name.endswith("f.b") else 0.0)
            else:
                t = 0.1 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * shape[-1] ** -0.5
            if leaf in ("i", "f"):
                t = t * 4.0
            if leaf == "router":
                t = t * 3.0
            if leaf == "embed":
                t = torch.randn(shape, generator=g)
        sd[name] = t.to(dtype)
    return sd
