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


# ----------------------------------------------------------------------------- small configurations and weights


def latent_layer(heads, dim, rot_dim, vdim, kv_rank, scale, base, mlp, **more):
    return {"type": "latent_attention", "mlp": mlp, **more,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim}}}


def delta_layer(heads, kv_heads, dim, vdim, conv, mlp, **more):
    return {"type": "channel_delta", "mlp": mlp, **more,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def moe(experts, identity, top, groups, keep, ff, limit, shared=None):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}},
            "shared": shared}


def model_config(vocab, width, eps, layers):
    return {"architecture": "Lemesun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


_MOE_A = moe(6, 2, 3, 4, 2, 24, 1.0, {"ff": 40, "limit": 0.7})
_MOE_B = moe(3, 0, 1, 1, 1, 20, 2.5)
# A: both mixers, a layer run twice, a layer without feed-forward, identity outputs, groups, a shared expert,
#    grouped q/k heads, a value size beyond one block of columns
TINY_A = model_config(97, 48, 1e-5, [
    latent_layer(3, 8, 4, 12, 20, 0.3, 100.0, _MOE_A),
    delta_layer(4, 2, 16, 8, 3, _MOE_A),
    latent_layer(3, 8, 4, 12, 20, 0.3, 100.0, _MOE_A, weights_of=0),
    delta_layer(2, 2, 40, 36, 2, None),
    delta_layer(4, 2, 16, 8, 3, _MOE_A, weights_of=1)])
# B: sizes of one (one head, one tap, one group, top 1), no identity outputs, no shared expert, delta first
TINY_B = model_config(61, 64, 1e-6, [
    delta_layer(1, 1, 24, 16, 1, _MOE_B),
    latent_layer(1, 16, 8, 16, 24, 0.2, 5000.0, _MOE_B),
    delta_layer(3, 3, 72, 16, 4, _MOE_B)])
# one mixer alone, no feed-forward
ONLY_LATENT = model_config(53, 32, 1e-6, [latent_layer(4, 8, 8, 8, 16, 0.35, 1000.0, None)])
ONLY_DELTA = model_config(53, 32, 1e-6, [delta_layer(4, 2, 16, 12, 4, None)])
# heads of 48 + 16 = 64 lanes (the size of the tcgen05 prefill kernel), and a latent row of 21 + 6 lanes (no multiple of 4)
LATENT_64 = model_config(53, 64, 1e-6, [latent_layer(2, 48, 16, 32, 40, 0.125, 10000.0, None),
                                        latent_layer(3, 10, 6, 8, 21, 0.25, 300.0, None)])
BOTTLENECKS = (6, 10)     # widths of the decay and gate bottlenecks in every test model


def random_weights(cfg, seed, sharpen=1.0):
    """bfloat16 tensors under the checkpoint names; scales chosen so that every mechanism moves the logits.
    ``sharpen`` multiplies the query projections of latent attention (peaky softmax: a lost key shows)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(rows, cols, scale=1.0):
        return (torch.randn(rows, cols, generator=g) * scale / cols ** 0.5).to(torch.bfloat16)

    def vec(n, scale, shift=0.0):
        return (torch.randn(n, generator=g) * scale + shift).to(torch.bfloat16)

    w = {"embed": (torch.randn(cfg["vocab"], W, generator=g)).to(torch.bfloat16), "final.norm": vec(W, 0.1),
         "head": mat(cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = vec(W, 0.1)
        if layer["type"] == "latent_attention":
            H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[p + "mix.q"] = mat(H * (d + r), W, 2.0 * sharpen)
            w[p + "mix.dkv"] = mat(R + r, W, 2.0)
            w[p + "mix.dkv.norm"] = vec(R, 0.2, 1.0)
            w[p + "mix.uk"] = mat(H * d, R, 2.0)
            w[p + "mix.uv"] = mat(H * dv, R)
            w[p + "mix.o"] = mat(W, H * dv)
        else:
            H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = BOTTLENECKS
            for name, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                w[p + f"mix.{name}"] = mat(rows, W, 2.0)
                w[p + f"mix.{name}.conv"] = (torch.randn(rows, K, generator=g) * 0.6).to(torch.bfloat16)
            w[p + "mix.b"] = mat(H, W, 2.0)
            w[p + "mix.A_log"] = vec(H, 0.5, -1.0)
            w[p + "mix.norm"] = vec(dv, 0.2, 1.0)
            w[p + "mix.a1"] = mat(ra, W)
            w[p + "mix.a2"] = mat(H * d, ra, 2.0)
            w[p + "mix.dt_bias"] = vec(H * d, 1.0)
            w[p + "mix.g1"] = mat(rg, W)
            w[p + "mix.g2"] = mat(H * dv, rg, 2.0)
            w[p + "mix.o"] = mat(W, H * dv)
        f = layer.get("mlp")
        if f is None:
            continue
        w[p + "norm2"] = vec(W, 0.1)
        n_all = f["router"]["experts"] + f["router"]["identity"]
        w[p + "mlp.router"] = mat(n_all, W, 3.0)
        w[p + "mlp.correction"] = vec(n_all, 0.05)
        for e in range(f["router"]["experts"]):
            w[p + f"mlp.e{e}.gate"] = mat(f["expert"]["ff"], W, 2.0)
            w[p + f"mlp.e{e}.up"] = mat(f["expert"]["ff"], W, 2.0)
            w[p + f"mlp.e{e}.down"] = mat(W, f["expert"]["ff"], 2.0)
        if f.get("shared"):
            w[p + "mlp.shared.gate"] = mat(f["shared"]["ff"], W, 2.0)
            w[p + "mlp.shared.up"] = mat(f["shared"]["ff"], W, 2.0)
            w[p + "mlp.shared.down"] = mat(W, f["shared"]["ff"])
    return w


def random_prompts(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


def widened(weights, dtype=torch.float64):
    return {k: v.to(dtype) for k, v in weights.items()}


def random_config(seed):
    """A valid configuration with sizes drawn from odd values (widths off the multiples of 8, one head, heads that
    share q/k, one tap, rows that are no multiple of 4, identity outputs or none, one group or several)."""
    g = torch.Generator().manual_seed(1000 + seed)

    def pick(values):
        return values[int(torch.randint(0, len(values), (1,), generator=g))]

    def some_moe():
        groups, per = pick([1, 2, 3]), pick([2, 3, 4])
        n_all = groups * per
        identity = pick([0, 1, 2]) if n_all > 2 else 0
        keep = pick(list(range(1, groups + 1)))
        top = pick(list(range(1, min(keep * per, 4) + 1)))
        shared = {"ff": pick([8, 20, 36]), "limit": pick([0.5, 1.5, 4.0])} if pick([0, 1]) else None
        return moe(n_all - identity, identity, top, groups, keep, pick([12, 20, 36]), pick([0.6, 1.5, 3.0]), shared)

    width = pick([40, 52, 72, 100])
    layers = []
    for i in range(pick([2, 3, 4])):
        mlp = some_moe() if pick([0, 1, 1]) else None
        if pick([0, 1]):
            rot = pick([2, 4, 6, 8])
            layers.append(latent_layer(pick([1, 2, 3, 5]), pick([4, 12, 16, 20]), rot, pick([4, 12, 20]),
                                       pick([9, 16, 22, 40]), pick([0.1, 0.3, 0.5]), pick([50.0, 10000.0, 1e6]), mlp))
        else:
            kv = pick([1, 2, 3])
            layers.append(delta_layer(kv * pick([1, 2]), kv, pick([6, 12, 33, 48]), pick([5, 16, 40]), pick([1, 2, 3, 5]), mlp))
    # one more run of an earlier layer's tensors, with a cache or state of its own
    source = pick(list(range(len(layers))))
    layers.append({**layers[source], "weights_of": source})
    return model_config(pick([31, 64, 101]), width, pick([1e-6, 1e-5]), layers)
