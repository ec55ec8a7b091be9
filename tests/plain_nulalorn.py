"""A plain, slow restatement of the Nulalorn decoder for tests: one function per mechanism, whole sequences at
a time, float64 on the CPU, no cache, no batching.  It shares no code with the library.

A model is ``(config, tensors)``: the ``config.json`` dictionary and a dictionary name -> tensor.

Notation.  T tokens, D = width.  Layer: x += n1b(mix(n1(x))); x += n2b(ff(n2(x))), n(.) an RMS norm with a weight.
Looped layers start..stop-1 run ``times`` times; before each pass x = W_in [x ; x0] + step[t], x0 the embedding.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    """Rows of x divided by sqrt(mean of squares + eps), times the weight (None: no weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` (factor, low, high, original) long wavelengths are
    slowed: wavelength above original/low -> f/factor, below original/high -> f, between them a blend."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f:
            wavelength = 2.0 * math.pi / fi
            if wavelength < original / high:
                out.append(fi)
            elif wavelength > original / low:
                out.append(fi / factor)
            else:
                s = (original / wavelength - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=F64)


def rotate_pairs(x, positions, freqs):
    """x [T, heads, dim]: lanes (2i, 2i+1), i < len(freqs), turn by positions * freqs[i]; other lanes pass."""
    out = x.clone()
    n = freqs.numel()
    angle = positions.to(F64)[:, None] * freqs[None, :]                  # [T, n]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = u * cos - v * sin
    out[..., 1:2 * n:2] = v * cos + u * sin
    return out


def visible(T, window):
    """[T, T] bool: query i sees key j when 0 <= i - j < window (window None: every j <= i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok &= (i - j) < window
    return ok


def capped_scores(q, k, scale, softcap):
    """q [T, d], k [T, d] -> [T, T] scores times scale, squashed by softcap * tanh(. / softcap) if given."""
    s = (q @ k.T) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    return s


def attention_mixer(h, tensors, prefix, m, eps, positions=None):
    """The design's attention on a whole sequence h [T, D]; ``m`` is the layer's ``mixer`` dictionary."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    if positions is None:
        positions = torch.arange(T)
    q = (h @ tensors[prefix + "q"].T).view(T, H, d)
    k = (h @ tensors[prefix + "k"].T).view(T, G, d)
    v = (h @ tensors[prefix + "v"].T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        freqs = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_pairs(q, positions, freqs), rotate_pairs(k, positions, freqs)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    window = (m.get("mask") or {}).get("size")
    see = visible(T, window)
    heads = []
    for head in range(H):
        g = head // (H // G)
        s = capped_scores(q[:, head], k[:, g], m["scale"], m.get("softcap"))
        s = s.masked_fill(~see, float("-inf"))
        heads.append(torch.softmax(s, -1) @ v[:, g])
    return torch.cat(heads, -1) @ tensors[prefix + "o"].T


def dense_ff(h, tensors, prefix):
    return gelu_erf(h @ tensors[prefix + "up"].T) @ tensors[prefix + "down"].T


def table_experts(h, token_ids, tensors, prefix, f):
    """Mixture of experts whose choice is a table row per token id, each chosen expert weighted 1/top, plus a
    shared expert times sigmoid(sg . h) when the layer has one."""
    top = f["router"]["top"]
    table = tensors[prefix + "table"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[int(token_ids[t])].tolist():
            out[t] += dense_ff(h[t:t + 1], tensors, f"{prefix}e{int(e)}.")[0] / top
    if f.get("shared"):
        gate = torch.sigmoid(h @ tensors[prefix + "shared.sg"].T)                    # [T, 1]
        out = out + gate * dense_ff(h, tensors, prefix + "shared.")
    return out


def layer(x, token_ids, tensors, i, entry, eps, positions=None):
    p = f"l{i}."
    if entry["type"] != "attention":
        raise ValueError(entry["type"])
    mixed = attention_mixer(rms_norm(x, tensors[p + "norm1"], eps), tensors, p + "mix.", entry["mixer"], eps, positions)
    x = x + rms_norm(mixed, tensors[p + "norm1b"], eps)
    f = entry.get("mlp")
    if f is not None:
        h = rms_norm(x, tensors[p + "norm2"], eps)
        if f["kind"] == "dense":
            y = dense_ff(h, tensors, p + "mlp.")
        else:
            y = table_experts(h, token_ids, tensors, p + "mlp.", f)
        x = x + rms_norm(y, tensors[p + "norm2b"], eps)
    return x


def layer_runs(config):
    """The executions in order: (layer index, pass number or None when the run does not open a pass)."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(config, tensors, token_ids, positions=None):
    """(logits [T, vocab], residual stream after every layer run [runs, T, D]) of one whole sequence."""
    tensors = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    x0 = tensors["embed"][ids]
    x = x0.clone()
    streams = []
    for i, opens in layer_runs(config):
        if opens is not None:
            x = torch.cat([x, x0], -1) @ tensors["loop.in"].T + tensors["loop.step"][opens]
        x = layer(x, ids, tensors, i, config["layers"][i], eps, positions)
        streams.append(x)
    logits = rms_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, torch.stack(streams)
