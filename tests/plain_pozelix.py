"""A plain, slow implementation of the Pozelix design: float64, no cache, whole sequences, one function per mechanism.

Written from the design's equations and sharing no code with the package. ``cfg`` is the configuration as a plain
dict (the keys of config.json), ``w`` maps tensor names to float64 tensors.

    layer:   x <- x + norm_b(mixer(norm_a(x)));  x <- x + norm_d(ff(norm_c(x)))      (norms before AND after a branch)
    loop:    layers start .. stop-1 run ``times`` times with the same weights; ahead of every pass
             x <- W_in [x ; x0], x0 the embedding output
    mixers:  grouped-query attention through a sliding window (rotation by halves, unit-norm q and k after the
             rotation, one sigmoid gate per head) and latent attention (queries through a normed latent, keys and
             values as up-projections of a normed latent, one rotated key part shared by the heads, rotation of
             neighbouring pairs with rescaled frequencies)
    ff:      gated SiLU unit, dense or as routed experts (softmax over all experts, choice by score + correction,
             weights the scores themselves, identity experts that return their input)
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis; weight None: no weight."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def frequencies(dims, base, scaling=None):
    """(f [dims/2], magnitude): angle of pair i at position p is p * f[i]; cos and sin are multiplied by magnitude."""
    i = torch.arange(dims // 2, dtype=F64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turns_to_dim(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns_to_dim(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, dims, base, pairing, scaling=None):
    """x [tokens, heads, width]: the first ``dims`` entries of every head are rotated. pairing "half": entry i with
    i + dims/2; "neighbours": entry 2i with 2i + 1."""
    if dims == 0:
        return x
    f, mag = frequencies(dims, base, scaling)
    ang = positions.to(F64)[:, None] * f[None, :]
    c, s = (ang.cos() * mag)[:, None, :], (ang.sin() * mag)[:, None, :]
    out = x.clone()
    if pairing == "half":
        u, v = x[..., : dims // 2], x[..., dims // 2: dims]
        out[..., : dims // 2] = u * c - v * s
        out[..., dims // 2: dims] = v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale, window):
    """q [T, H, d], k [T, H, d], v [T, H, dv] (keys already per query head). Position i sees j <= i, and with a
    window > 0 only i - j < window."""
    T = q.shape[0]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window > 0:
        seen = seen & (i - j < window)
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v)


def window_attention(h, m, w, p, eps):
    """The mixer 'attention'. h [T, width]; m: the mixer's configuration; p: the tensors' prefix."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    rot = m.get("rot") or {}
    dims = rot.get("dims", 0)
    q = rotate(q, pos, dims, rot.get("base", 1.0), "half", rot.get("scaling"))
    k = rotate(k, pos, dims, rot.get("base", 1.0), "half", rot.get("scaling"))
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    window = (m.get("mask") or {}).get("size", 0)
    o = softmax_attention(q, k, v, m["scale"], window)
    gate = torch.sigmoid(h @ w[p + "g"].T)               # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def latent_attention(h, m, w, p, eps):
    """The mixer 'latent_attention'."""
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    rot = m["rot"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, d + dr)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    kr = down[:, rank:].view(T, 1, dr)
    qr = rotate(q[..., d:], pos, dr, rot["base"], "neighbours", rot.get("scaling"))
    kr = rotate(kr, pos, dr, rot["base"], "neighbours", rot.get("scaling"))
    kn = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    qq = torch.cat([q[..., :d], qr], dim=-1)
    kk = torch.cat([kn, kr.expand(T, H, dr)], dim=-1)
    o = softmax_attention(qq, kk, v, m["scale"], (m.get("mask") or {}).get("size", 0))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def gated_unit(h, w, p):
    g = h @ w[p + "gate"].T
    return ((g * torch.sigmoid(g)) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, f, w, p):
    """(chosen [T, top], weights [T, top]): softmax over all experts (identity ones included), choice by
    score + correction, weights the scores themselves."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    chosen = torch.topk(s + w[p + "correction"], f["router"]["top"], dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def routed_experts(h, f, w, p):
    n, ident = f["router"]["experts"], f["router"].get("identity", 0)
    chosen, weights = route(h, f, w, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            if e >= n:
                assert e < n + ident
                out[t] += a * h[t]
            else:
                out[t] += a * gated_unit(h[t: t + 1], w, f"{p}e{e}.")[0]
    return out


def feed_forward(h, f, w, p):
    return gated_unit(h, w, p) if f["kind"] == "dense" else routed_experts(h, f, w, p)


def layer(x, i, cfg, w):
    eps = cfg["norm"]["eps"]
    L, p = cfg["layers"][i], f"l{i}."
    mixer = {"attention": window_attention, "latent_attention": latent_attention}[L["type"]]
    a = mixer(rms_norm(x, w[p + "norm1"], eps), L["mixer"], w, p + "mix.", eps)
    x = x + rms_norm(a, w[p + "norm1b"], eps)
    if L.get("mlp") is not None:
        b = feed_forward(rms_norm(x, w[p + "norm2"], eps), L["mlp"], w, p + "mlp.")
        x = x + rms_norm(b, w[p + "norm2b"], eps)
    return x


def run_order(cfg):
    """[(layer, starts a pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(tokens, cfg, w, residuals=None):
    """Logits [T, vocab] of one sequence. ``residuals``: a list that receives the stream after every layer run."""
    x0 = w["embed"][torch.as_tensor(tokens)]
    x = x0
    for i, enters in run_order(cfg):
        if enters:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        x = layer(x, i, cfg, w)
        if residuals is not None:
            residuals.append(x)
    return rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T


def load_model_dir(path: str):
    """(config dict, {name: float64 tensor}) of a model folder."""
    import json
    import os

    from plain_rusadra import read_safetensors
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(path, "model.safetensors"))
    return cfg, {k: v.to(F64) for k, v in w.items()}
