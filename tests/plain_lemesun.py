"""A plain, slow restatement of the Lemesun decoder: one function per mechanism, whole sequences, no cache.

Everything runs on the CPU in the dtype of the tensors it is given (the tests use float64 or float32) and shares
no code with the library.  ``cfg`` is the ``config.json`` dictionary and ``w`` a dictionary of tensors by
checkpoint name.

Notation: T tokens, positions 0..T-1; x [T, width] is the residual stream.
"""

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return rms(x, eps) * (1.0 + weight)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x, positions, base, dims):
    """Rotate lanes (2i, 2i+1), i < dims/2, of the last axis of x [T, ..., d] by positions * base^(-2i/dims)."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_attention(h, w, p, m, eps, positions=None):
    """h [T, width] (normed input); p the tensor prefix ('l0.mix.'); m the mixer's config entry."""
    T = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], q[..., d:]
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :R], eps) * w[p + "dkv.norm"]
    k_rot = down[:, R:]
    q_rot = rotate_pairs(q_rot, pos, m["rot"]["base"], m["rot"]["dims"])
    k_rot = rotate_pairs(k_rot, pos, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    scores = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)
    scores = scores * m["scale"]
    visible = pos[None, :] <= pos[:, None]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    o = torch.einsum("hij,jhd->ihd", torch.softmax(scores, -1), v).reshape(T, H * dv)
    return o @ w[p + "o"].T


def causal_conv_silu(x, taps):
    """x [T, C], taps [C, K] (last column: the current token); zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j][None, :]
    return torch.nn.functional.silu(y)


def channel_delta(h, w, p, m, eps):
    """The gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"]).view(T, G, d)
    k = causal_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"]).view(T, G, d)
    v = causal_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                        # [T, H]
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]                    # [T, H*d]
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * torch.nn.functional.softplus(a).view(T, H, d))
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        src = head // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, src])
            S = S + torch.outer(k[t, src], u)
            out[t, head] = S.T @ q[t, src]
    out = rms(out, eps) * w[p + "norm"] * gate
    return out.reshape(T, H * dv) @ w[p + "o"].T


def clamped_expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, w, p, f):
    """(chosen [T, top], weights [T, top]) of the grouped top-k router."""
    r = f["router"]
    n_all = r["experts"] + r["identity"]
    s = torch.softmax(h @ w[p + "router"].T, -1)
    choice = s + w[p + "correction"]
    groups, keep = r["groups"]["count"], r["groups"]["keep"]
    per = n_all // groups
    best = choice.view(-1, groups, per).max(-1).values
    kept = best.topk(keep, -1).indices
    allowed = torch.zeros(h.shape[0], groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    choice = choice.masked_fill(~allowed.repeat_interleave(per, 1), float("-inf"))
    chosen = choice.topk(r["top"], -1).indices
    return chosen, s.gather(1, chosen)


def mixture(h, w, p, f):
    r = f["router"]
    chosen, weight = route(h, w, p, f)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), weight[t]):
            if e >= r["experts"]:
                out[t] += s * h[t]
            else:
                q = f"{p}e{e}."
                out[t] += s * clamped_expert(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"], f["expert"]["limit"])[0]
    if f.get("shared"):
        q = p + "shared."
        out = out + clamped_expert(h, w[q + "gate"], w[q + "up"], w[q + "down"], f["shared"]["limit"])
    return out


def forward(cfg, w, ids, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer run if asked)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(ids)]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        h = offset_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            x = x + latent_attention(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "channel_delta":
            x = x + channel_delta(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + mixture(offset_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
        after.append(x)
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if keep_layers else logits
