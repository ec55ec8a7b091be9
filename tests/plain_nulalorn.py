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


# ------------------------------------------------------------------------------ small models for the tests


def attention_layer(*, heads, kv_heads, dim, vdim, scale, softcap=None, window=None, rot=None, mlp=None):
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if softcap is not None:
        mixer["softcap"] = softcap
    if window is not None:
        mixer["mask"] = {"size": window}
    if rot is not None:
        mixer["rot"] = rot
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def moe(experts, top, ff, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


SCALED = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}      # at base 100, 8 lanes: keep, blend, blend, slow

# A: a dense layer, then two layers with experts that run three times, then a layer without feed-forward.
TINY_A = {
    "architecture": "Nulalorn", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        attention_layer(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.4, softcap=9.0, window=7,
                        rot={"base": 100.0, "dims": 8, "scaling": SCALED}, mlp={"kind": "dense", "ff": 72}),
        attention_layer(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.4, softcap=9.0, window=7,
                        rot={"base": 100.0, "dims": 8, "scaling": SCALED}, mlp=moe(5, 2, 24, shared=40)),
        attention_layer(heads=2, kv_heads=1, dim=32, vdim=24, scale=0.25, softcap=5.0, window=70,
                        rot={"base": 1000.0, "dims": 32}, mlp=moe(3, 1, 32)),
        attention_layer(heads=4, kv_heads=4, dim=16, vdim=16, scale=0.3, window=3, rot={"base": 50.0, "dims": 2}),
    ],
}

# B: values that may be one or equal elsewhere are not here: every head its own key/value head, a value as wide as
# a key, one expert per token, the loop from the first layer on, a layer that sees every key, no cap on the logits.
TINY_B = {
    "architecture": "Nulalorn", "vocab": 45, "width": 40, "norm": {"eps": 1e-6},
    "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [
        attention_layer(heads=3, kv_heads=3, dim=12, vdim=12, scale=0.5, rot={"base": 300.0, "dims": 12},
                        mlp=moe(4, 1, 16, shared=8)),
        attention_layer(heads=5, kv_heads=1, dim=8, vdim=20, scale=0.6, softcap=4.0, window=64, mlp={"kind": "dense", "ff": 56}),
    ],
}

# C: odd sizes: a width off the multiples of 8, heads of 6 lanes (stored as 8), values of 5, six query heads on one
# key/value head, a window of one (a token sees itself only), three experts of five, a loop over all layers, run once.
TINY_C = {
    "architecture": "Nulalorn", "vocab": 33, "width": 44, "norm": {"eps": 1e-4}, "logit_softcap": 3.0,
    "loop": {"start": 0, "stop": 2, "times": 1},
    "layers": [
        attention_layer(heads=6, kv_heads=1, dim=6, vdim=5, scale=0.9, softcap=2.5, window=1,
                        rot={"base": 10.0, "dims": 6, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16}},
                        mlp=moe(5, 3, 12, shared=20)),
        attention_layer(heads=2, kv_heads=2, dim=20, vdim=4, scale=0.35, softcap=30.0, window=130,
                        rot={"base": 10000.0, "dims": 4}, mlp={"kind": "dense", "ff": 30}),
    ],
}

# SHARP: one looped layer whose scores reach scale * dim = 24 before a cap of 40: the softmax picks single keys
# anywhere inside a window of 300 positions (several pages), so a lost or misplaced far key moves the logits.
SHARP = {
    "architecture": "Nulalorn", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
    "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [attention_layer(heads=2, kv_heads=1, dim=16, vdim=16, scale=1.5, softcap=40.0, window=300,
                               rot={"base": 10000.0, "dims": 8}, mlp={"kind": "dense", "ff": 48})],
}

# WIDE_HEADS: key and value heads of 64 lanes (the sizes of the kernel that keeps scores in tensor memory), a window
# that crosses pages, a second layer that sees every key.
WIDE_HEADS = {
    "architecture": "Nulalorn", "vocab": 70, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 15.0,
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [attention_layer(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.2, softcap=12.0, window=100,
                               rot={"base": 10000.0, "dims": 32, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}},
                               mlp=moe(4, 2, 32, shared=32)),
               attention_layer(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.15, rot={"base": 500.0, "dims": 64},
                               mlp={"kind": "dense", "ff": 96})],
}

# NOLOOP: no loop at all and nothing optional.
PLAIN_STACK = {
    "architecture": "Nulalorn", "vocab": 29, "width": 24, "norm": {"eps": 1e-5},
    "layers": [attention_layer(heads=2, kv_heads=2, dim=8, vdim=8, scale=0.35, mlp={"kind": "dense", "ff": 40}),
               attention_layer(heads=1, kv_heads=1, dim=16, vdim=12, scale=0.25, window=9, mlp=moe(2, 2, 8))],
}


def tensor_shapes(config):
    """name -> shape of every tensor the design stores for ``config`` (an integer table: rows, entries per row, bound, 'int')."""
    D, V = config["width"], config["vocab"]
    shapes = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    if config.get("loop"):
        shapes["loop.in"] = (D, 2 * D)
        shapes["loop.step"] = (config["loop"]["times"], D)
    for i, entry in enumerate(config["layers"]):
        p, m = f"l{i}.", entry["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = (D,)
        shapes[p + "mix.q"] = (m["heads"] * m["dim"], D)
        shapes[p + "mix.k"] = (m["kv_heads"] * m["dim"], D)
        shapes[p + "mix.v"] = (m["kv_heads"] * m["vdim"], D)
        shapes[p + "mix.o"] = (D, m["heads"] * m["vdim"])
        f = entry.get("mlp")
        if f is None:
            continue
        shapes[p + "norm2"] = shapes[p + "norm2b"] = (D,)
        if f["kind"] == "dense":
            shapes[p + "mlp.up"], shapes[p + "mlp.down"] = (f["ff"], D), (D, f["ff"])
            continue
        for e in range(f["router"]["experts"]):
            shapes[f"{p}mlp.e{e}.up"], shapes[f"{p}mlp.e{e}.down"] = (f["expert"]["ff"], D), (D, f["expert"]["ff"])
        shapes[p + "mlp.table"] = (V, f["router"]["top"], f["router"]["experts"], "int")
        if f.get("shared"):
            shapes[p + "mlp.shared.up"], shapes[p + "mlp.shared.down"] = (f["shared"]["ff"], D), (D, f["shared"]["ff"])
            shapes[p + "mlp.shared.sg"] = (1, D)
    return shapes


def random_weights(config, seed):
    """Tensors as a checkpoint stores them (bfloat16, tables int32): matrices normal with a spread that keeps every
    activation of order one, norm weights around one, a table of distinct experts per token id."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        if shape[-1] == "int":
            rows = [torch.randperm(shape[2], generator=g)[:shape[1]] for _ in range(shape[0])]
            out[name] = torch.stack(rows).to(torch.int32)
        elif len(shape) == 1:
            out[name] = (1.0 + 0.2 * torch.randn(shape, generator=g)).to(torch.bfloat16)
        elif name in ("embed", "loop.step"):
            out[name] = torch.randn(shape, generator=g).to(torch.bfloat16)
        else:
            out[name] = (torch.randn(shape, generator=g) * (1.5 / shape[-1] ** 0.5)).to(torch.bfloat16)
    return out


def random_prompts(config, lengths, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in lengths]


def random_config(seed):
    """A configuration drawn from odd values: sizes, counts, windows, loop and optional mechanisms all vary."""
    g = torch.Generator().manual_seed(500 + seed)
    pick = lambda *values: values[int(torch.randint(0, len(values), (1,), generator=g))]
    width, vocab = pick(20, 36, 52, 64), pick(17, 40, 75)
    layers = []
    for _ in range(pick(1, 2, 3)):
        kv = pick(1, 2, 3)
        dim, half = pick(4, 10, 16, 24, 36), None
        rot = None
        if pick(True, True, False):
            rot = {"base": pick(10.0, 500.0, 10000.0), "dims": pick(2, 4, dim)}
            if pick(True, False):
                rot["scaling"] = {"factor": pick(2.0, 4.0), "low": 1.0, "high": pick(2.0, 4.0), "original": pick(8, 64, 512)}
        kind = pick("dense", "moe", "moe", None)
        mlp = None
        if kind == "dense":
            mlp = {"kind": "dense", "ff": pick(8, 28, 72)}
        elif kind == "moe":
            experts = pick(1, 2, 6, 9)
            mlp = moe(experts, pick(*range(1, min(experts, 3) + 1)), pick(8, 12, 40), shared=pick(None, 8, 24))
        layers.append(attention_layer(heads=kv * pick(1, 2, 4), kv_heads=kv, dim=dim, vdim=pick(3, 8, dim, 40),
                                      scale=pick(0.2, 0.5, 1.0) / dim ** 0.5 * 2, softcap=pick(None, 3.0, 25.0),
                                      window=pick(None, 1, 2, 33, 64, 65, 100), rot=rot, mlp=mlp))
    config = {"architecture": "Nulalorn", "vocab": vocab, "width": width, "norm": {"eps": pick(1e-6, 1e-5, 1e-3)}, "layers": layers}
    if pick(True, True, False):
        start = pick(*range(len(layers)))
        config["loop"] = {"start": start, "stop": pick(*range(start + 1, len(layers) + 1)), "times": pick(1, 2, 3)}
    if pick(True, False):
        config["logit_softcap"] = pick(2.0, 30.0)
    return config
