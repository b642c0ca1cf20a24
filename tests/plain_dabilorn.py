"""A plain, slow implementation of the Dabilorn design in float64: whole sequences, no cache, no state carried between calls,
one function per mechanism.  It shares no code with the engine; the tests compare the engine with it.

Notation: ``x`` [S, width] is a sequence's residual stream, ``h`` a sub-layer's input, ``W[name]`` a tensor of the model
folder (matrices are stored [out, in] and applied as ``h @ W.T``), ``m`` a layer's ``mixer`` object of config.json and ``f``
its ``mlp`` object.
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, w, eps):
    """No bias; the variance is the mean of the squared deviations."""
    c = x - x.mean(-1, keepdim=True)
    return c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


# ------------------------------------------------------------------------------------------ input convolution
def time_conv(h, w):
    """h [S, C], w [C, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the first token."""
    S, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for t in range(S):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                out[t] += w[:, j] * h[src]
    return out


# ------------------------------------------------------------------------------------------ rotations
def frequencies(rot):
    """The angle per position of every rotated pair, and what cosine and sine are multiplied by."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def turn(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(sc["fast"])), 0)
    hi = min(math.ceil(turn(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, rot, pairing):
    """x [S, heads, D]: the first rot.dims values of every head are turned by ``position * frequency``;
    ``pairing`` "interleaved": value 2i with value 2i + 1; "half": value i with value i + dims/2."""
    if not rot or not rot["dims"]:
        return x
    S, dims = x.shape[0], rot["dims"]
    f, mag = frequencies(rot)
    out = x.clone()
    for i in range(dims // 2):
        a, b = (2 * i, 2 * i + 1) if pairing == "interleaved" else (i, i + dims // 2)
        angle = torch.arange(S, dtype=F64) * f[i]
        c, s = (torch.cos(angle) * mag)[:, None], (torch.sin(angle) * mag)[:, None]
        out[:, :, a] = x[:, :, a] * c - x[:, :, b] * s
        out[:, :, b] = x[:, :, b] * c + x[:, :, a] * s
    return out


# ------------------------------------------------------------------------------------------ masks
def visible(S, chunk=None):
    """[S, S] bool: row i sees column j <= i, and with a chunk size only inside i's own chunk."""
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    ok = j <= i
    if chunk is not None:
        ok &= (i // chunk) == (j // chunk)
    return ok


# ------------------------------------------------------------------------------------------ latent attention
def latent_attention(h, W, p, m, eps):
    S = h.shape[0]
    H, D, R, Dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(S, H, D + R)
    dkv = h @ W[p + "dkv"].T
    c = rms_norm(dkv[:, :rank], eps) * W[p + "dkv.norm"]
    k_rot = rotate(dkv[:, rank:].reshape(S, 1, R), m.get("rot"), "interleaved")[:, 0]
    q_rot = rotate(q[:, :, D:].contiguous(), m.get("rot"), "interleaved")
    k_plain = (c @ W[p + "uk"].T).view(S, H, D)
    v = (c @ W[p + "uv"].T).view(S, H, Dv)
    mask = visible(S)
    heads = []
    for n in range(H):
        s = (q[:, n, :D] @ k_plain[:, n].T + q_rot[:, n] @ k_rot.T) * m["scale"]
        s = s.masked_fill(~mask, float("-inf"))
        heads.append(torch.softmax(s, dim=-1) @ v[:, n])
    o = torch.cat(heads, dim=-1) * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ sigmoid attention
def attention(h, W, p, m, eps):
    """Grouped heads, one RMS norm over all of q (and of k), rotated halves, chunked mask, sigmoid weights with a bias per head."""
    S = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ W[p + "q"].T, eps) * W[p + "q.norm"]
    k = rms_norm(h @ W[p + "k"].T, eps) * W[p + "k.norm"]
    v = (h @ W[p + "v"].T).view(S, G, Dv)
    q = rotate(q.view(S, H, D), m.get("rot"), "half")
    k = rotate(k.view(S, G, D), m.get("rot"), "half")
    mask = visible(S, (m.get("mask") or {}).get("size"))
    heads = []
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].T) * m["scale"]
        w = sigmoid(s + W[p + "pb"][n]) * mask
        heads.append(w @ v[:, g])
    o = torch.cat(heads, dim=-1) * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ time mixing
def wkv(h, W, p, m, eps):
    S = h.shape[0]
    H, D = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def mix(s):
        return h + (prev - h) * W[p + "mu." + s]

    r = (mix("r") @ W[p + "r"].T).view(S, H, D)
    k = (mix("k") @ W[p + "k"].T).view(S, H, D)
    v = (mix("v") @ W[p + "v"].T).view(S, H, D)
    gz = mix("g") @ W[p + "g"].T
    gate = gz * sigmoid(gz)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).view(S, H, D)
    u = W[p + "u"].view(H, D)
    out = torch.zeros(S, H, D, dtype=F64)
    for n in range(H):
        state = torch.zeros(D, D, dtype=F64)                      # [key channel, value channel]
        for t in range(S):
            kv = k[t, n][:, None] * v[t, n][None, :]
            out[t, n] = (state + u[n][:, None] * kv).T @ r[t, n]
            state = decay[t, n][:, None] * state + kv
    o = rms_norm(out, eps).reshape(S, H * D) * W[p + "norm"] * gate
    return o @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ feed-forward
def expert(h, W, p):
    return torch.relu(h @ W[p + "up"].T) ** 2 @ W[p + "down"].T


def moe(h, W, p, f):
    S = h.shape[0]
    s = sigmoid(h @ W[p + "router"].T)
    out = torch.zeros_like(h)
    for t in range(S):
        for e in torch.topk(s[t], f["router"]["top"]).indices.tolist():
            out[t] += expert(s[t, e] * h[t:t + 1], W, f"{p}e{e}.")[0]
    if f.get("shared"):
        out = out + expert(h, W, p + "shared.") * sigmoid(h @ W[p + "shared.sg"].T)
    return out


# ------------------------------------------------------------------------------------------ the model
MIXERS = {"latent_attention": latent_attention, "attention": attention, "wkv": wkv}


def forward(config, weights, tokens, after_layer=None):
    """Logits [S, vocab] (float64) of one whole sequence.  ``after_layer(i, x)`` sees the stream behind every layer."""
    W = {k: v.to(F64) for k, v in weights.items() if v.is_floating_point()}
    eps = config["norm"]["eps"]
    x = layer_norm(W["embed"][torch.as_tensor(tokens, dtype=torch.long)], W["embed.norm"], eps)
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        h = x + time_conv(x, W[p + "canon1"]) if config.get("canon") else x
        a = MIXERS[L["type"]](h, W, p + "mix.", L["mixer"], eps)
        x = x + layer_norm(a, W[p + "norm1"], eps) * W[p + "ls1"]
        if L.get("mlp") is not None:
            x = x + layer_norm(moe(x, W, p + "mlp.", L["mlp"]), W[p + "norm2"], eps) * W[p + "ls2"]
        if after_layer is not None:
            after_layer(i, x)
    return layer_norm(x, W["final.norm"], eps) @ W["embed"].T
