"""A plain, slow implementation of the Fekolorn design: float64, no cache, whole sequences, one function per mechanism.

Written from the design's equations and sharing no code with the package. ``cfg`` is the configuration as a plain
dict (the keys of config.json), ``w`` maps tensor names to float64 tensors.

    embedding  x = E[token] * scale + B[(prev * mul_prev + token * mul_cur) mod buckets]; the first token of a sequence
               takes row number ``buckets`` of B
    streams    s copies of x; a sublayer reads u = sum_s in[s] x_s, makes y = sublayer(norm(u)), and every stream becomes
               x_t <- sum_s mix[s, t] x_s + out[t] y; the model's output is the sum of the streams. With one stream and
               no such tensors this is x <- x + sublayer(norm(x)).
    norm       x / sqrt(mean(x^2) + eps) * g with ONE number g
    mixers     "parallel": softmax attention (rotation of a head's first channels by halves, values brought to unit
               root mean square, a sink) beside a gated delta rule (short causal convolutions, unit q and k, a scalar
               decay and a write strength per head), weighted sum of the two;
               "attention": norm over the whole q and k rows, no rotation, a learned bias per distance bucket and head,
               a sliding window, a sink, values mixed with those of the first such layer
    ff         W_down act(W_up h) with act = a N(z) + b N(z^2) + c N(z^3) + e, N the division by the root mean square
"""
import json
import math
import os
import struct

import torch

F64 = torch.float64


def rms(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def embed(tokens, cfg, w):
    e = cfg["embedding"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][ids] * float(e.get("scale", 1.0))
    b = e.get("bigram")
    if b:
        rows = torch.empty_like(ids)
        rows[0] = b["buckets"]
        rows[1:] = (ids[:-1] * b["mul_prev"] + ids[1:] * b["mul_cur"]) % b["buckets"]
        x = x + w["bigram"][rows]
    return x


def rotate_halves(x, positions, dims, base):
    """x [T, heads, width]: entry i of a head is paired with entry i + dims/2, for i < dims/2; the rest passes."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=F64)
    ang = positions.to(F64)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., : dims // 2], x[..., dims // 2: dims]
    out = x.clone()
    out[..., : dims // 2] = u * c - v * s
    out[..., dims // 2: dims] = v * c + u * s
    return out


def distance_bucket(n, rows, far):
    """Bucket of distance n >= 0 among ``rows`` buckets: the first half one per distance, the second half spaced by
    the logarithm up to distance ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def softmax_with_sink(scores, seen, sink):
    """scores [H, T, T], seen [T, T] bool, sink [H] or None: weights whose denominator also holds exp(sink_h)."""
    s = scores.masked_fill(~seen[None], float("-inf"))
    if sink is None:
        return torch.softmax(s, dim=-1)
    H, T, _ = s.shape
    s = torch.cat([s, sink.view(H, 1, 1).expand(H, T, 1)], dim=-1)
    return torch.softmax(s, dim=-1)[..., :-1]


def softmax_mixer(h, m, w, p, eps, positions, whole_norm, value_norm, v_first=None):
    """The softmax attention of both mixers. ``whole_norm``: q and k are normed over the whole projection with weights;
    ``value_norm``: every head's value is brought to unit root mean square; a rotation is applied when the mixer names
    one; with ``bias_max`` a distance bias; with ``mask.size`` a window. Returns (W_o's output, the values as cached)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if whole_norm:
        q = rms(q, eps) * w[p + "q.norm"]
        k = rms(k, eps) * w[p + "k.norm"]
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_halves(q, positions, rot["dims"], rot["base"])
        k = rotate_halves(k, positions, rot["dims"], rot["base"])
    if value_norm:
        v = rms(v, eps)                              # cached so
    if m.get("v_mix") and v_first is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    cached_v = v
    rep = H // G
    k, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    i, j = positions[:, None], positions[None, :]
    seen = j <= i
    if "bias_max" in m:
        rel = w[p + "rel"]
        rows = rel.shape[0]
        dist = (i - j).clamp(min=0)
        bucket = torch.tensor([[distance_bucket(int(n), rows, m["bias_max"]) for n in row] for row in dist.tolist()])
        s = s + rel[bucket].permute(2, 0, 1)
    size = (m.get("mask") or {}).get("size", 0)
    if size:
        seen = seen & (i - j < size)
    a = softmax_with_sink(s, seen, w.get(p + "sink"))
    o = torch.einsum("hij,jhd->ihd", a, vv).reshape(T, H * dv)
    return o @ w[p + "o"].T, cached_v


def short_conv(x, taps):
    """x [T, C], taps [C, K]: y_t = sum_j taps[:, K-1-j] x_(t-j), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([x.new_zeros((K - 1, C)), x], dim=0)
    y = x.new_zeros((T, C))
    for j in range(K):
        y = y + padded[j: j + T] * taps[:, j]
    return y


def gated_delta(h, m, w, p, eps):
    """The recurrent half: per head S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    unit = lambda x: x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)
    q, k = unit(q) * d ** -0.5, unit(k)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                                   # [T, H]
    g = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    rep = H // G
    out = h.new_zeros((T, H, dv))
    for hd in range(H):
        S = h.new_zeros((d, dv))
        for t in range(T):
            kt, qt = k[t, hd // rep], q[t, hd // rep]
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ kt)
            S = S + torch.outer(kt, u)
            out[t, hd] = S.T @ qt
    out = rms(out, eps) * w[p + "norm"]
    out = out.reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def parallel_mixer(h, m, w, p, eps, positions, v_first=None):
    """(weighted sum of the two sides, the softmax side's values as cached)."""
    left, cached = softmax_mixer(h, m["left"], w, p + "left.", eps, positions, whole_norm=False, value_norm=True,
                                 v_first=v_first)
    right = gated_delta(h, m["right"], w, p + "right.", eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right, cached


def poly_norm(z, coeff, eps):
    a, b, c, e = (coeff[i] for i in range(4))
    return a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e


def feed_forward(h, f, w, p, eps):
    return poly_norm(h @ w[p + "up"].T, w[p + "act"], eps) @ w[p + "down"].T


def scalar_norm(x, g, eps):
    return rms(x, eps) * g


def sublayer(streams, fn, norm_g, eps, w, hc):
    """One sublayer over the streams [s, T, D]: with hyper-connection tensors under ``hc`` the read, the mix and the
    write; without them (one stream) the plain residual sum."""
    if hc + "in" not in w:
        return streams + fn(scalar_norm(streams[0], norm_g, eps))[None]
    u = torch.einsum("s,std->td", w[hc + "in"], streams)
    y = fn(scalar_norm(u, norm_g, eps))
    return torch.einsum("sr,std->rtd", w[hc + "mix"], streams) + w[hc + "out"][:, None, None] * y[None]


def forward(tokens, cfg, w, residuals=None):
    """Logits [T, vocab] of one sequence. ``residuals`` (a list) receives the sum of the streams after every layer."""
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x0 = embed(tokens, cfg, w)
    streams = x0[None].repeat(int(cfg.get("streams", 1)), 1, 1)
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        kept = {}
        if layer["type"] == "parallel":
            softmax = m["left"]

            def fn(h, kept=kept, m=m):
                o, kept["v"] = parallel_mixer(h, m, w, p + "mix.", eps, positions, v_first=v_first)
                return o
        else:
            softmax = m

            def fn(h, kept=kept, m=m):
                o, kept["v"] = softmax_mixer(h, m, w, p + "mix.", eps, positions, whole_norm=True, value_norm=False,
                                             v_first=v_first)
                return o
        streams = sublayer(streams, fn, w[p + "norm1"], eps, w, p + "hc1.")
        if softmax.get("v_mix") and v_first is None:
            v_first = kept["v"]      # the first such layer's values, which it keeps unmixed
        if layer.get("mlp") is not None:
            f = layer["mlp"]
            streams = sublayer(streams, lambda h: feed_forward(h, f, w, p + "mlp.", eps), w[p + "norm2"], eps, w,
                               p + "hc2.")
        if residuals is not None:
            residuals.append(streams.sum(dim=0))
    x = scalar_norm(streams.sum(dim=0), w["final.norm"], eps)
    return x @ w["head"].T


def load_model_dir(path: str):
    """(cfg, tensors as float64) of a folder with config.json and model.safetensors (own reader: 8-byte length,
    JSON header, data)."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64}
    w = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        w[name] = t.to(F64) if t.is_floating_point() else t
    return cfg, w
