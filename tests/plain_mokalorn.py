"""A plain, slow implementation of the Mokalorn design in float64: whole sequences, no cache, no state carried between calls,
one function per mechanism.  It shares no code with the engine; the tests compare the engine with it.

Notation: ``x`` [S, width] is a sequence's residual stream, ``h`` a sub-layer's normed input, ``W[name]`` a tensor of the
model folder (matrices are stored [out, in] and applied as ``h @ W.T``), ``m`` a layer's ``mixer`` object of config.json and
``f`` its ``mlp`` object.
"""
import math

import torch

F64 = torch.float64
GLU_ALPHA, GLU_SHIFT = 1.702, 1.0


def rms_norm(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ------------------------------------------------------------------------------------------ rotations
def rotate(x, rot, pairing):
    """x [S, heads, D]: the first rot.dims values of every head are turned by ``position * base^(-2i/dims)``;
    ``pairing`` "interleaved": value 2i with value 2i + 1; "half": value i with value i + dims/2."""
    if not rot or not rot["dims"]:
        return x
    S, dims = x.shape[0], rot["dims"]
    out = x.clone()
    for i in range(dims // 2):
        a, b = (2 * i, 2 * i + 1) if pairing == "interleaved" else (i, i + dims // 2)
        angle = torch.arange(S, dtype=F64) * rot["base"] ** (-2.0 * i / dims)
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        out[:, :, a] = x[:, :, a] * c - x[:, :, b] * s
        out[:, :, b] = x[:, :, b] * c + x[:, :, a] * s
    return out


# ------------------------------------------------------------------------------------------ softmax attention
def visible(S, chunk):
    """[S, S] bool: row i sees column j <= i, and with a chunk size only inside i's own chunk."""
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    ok = j <= i
    if chunk is not None:
        ok &= (i // chunk) == (j // chunk)
    return ok


def softmax_heads(q, k, v, scale, mask):
    """q [S, H, D], k [S, G, D], v [S, G, Dv] -> [S, H * Dv]; query head h reads key/value head h // (H / G)."""
    S, H, _ = q.shape
    G = k.shape[1]
    outs = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        outs.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.cat(outs, dim=-1)


def query_temperature(S, q_temp):
    p = torch.arange(S, dtype=F64)
    return 1.0 + q_temp["coef"] * torch.log(torch.floor((p + 1.0) / q_temp["every"]) + 1.0)


def attention(h, W, p, m, eps, kind):
    """``kind`` "attention": the values are the projected keys (before norm and rotation), interleaved rotation, chunked mask.
    ``kind`` "attention_2": a value projection, no rotation, a query temperature that grows with the position, causal mask."""
    S = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W[p + "q"].T).view(S, H, D)
    k = (h @ W[p + "k"].T).view(S, G, D)
    if kind == "attention":
        v = k.clone()
    else:
        v = (h @ W[p + "v"].T).view(S, G, m["vdim"])
    q = rms_norm(q, eps) * W[p + "q.norm"]
    k = rms_norm(k, eps) * W[p + "k.norm"]
    if kind == "attention":
        q, k = rotate(q, m.get("rot"), "interleaved"), rotate(k, m.get("rot"), "interleaved")
        mask = visible(S, m["mask"]["size"] if m.get("mask") else None)
    else:
        if m.get("q_temp"):
            q = q * query_temperature(S, m["q_temp"])[:, None, None]
        mask = visible(S, None)
    o = softmax_heads(q, k, v, m["scale"], mask)
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ retention
def retention(h, W, p, m, eps):
    S = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = rotate((h @ W[p + "q"].T).view(S, H, D), m.get("rot"), "half")
    k = rotate((h @ W[p + "k"].T).view(S, H, D), m.get("rot"), "half") * D ** -0.5
    v = (h @ W[p + "v"].T).view(S, H, Dv)
    out = torch.zeros(S, H, Dv, dtype=F64)
    for hd in range(H):
        state = torch.zeros(D, Dv, dtype=F64)
        for t in range(S):
            state = m["decay"][hd] * state + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = state.T @ q[t, hd]
    out = rms_norm(out, eps).reshape(S, H * Dv)
    g = h @ W[p + "g"].T
    return (out * g * torch.sigmoid(g)) @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ feed-forward
def expert(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(GLU_ALPHA * g) * (u + GLU_SHIFT)) @ W[p + "down"].T


def route(h, W, p, f):
    """(chosen experts [S, top], their weights [S, top]); the router's last ``identity`` outputs are identity experts."""
    r = f["router"]
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    choice = s + W[p + "correction"]
    idx = torch.topk(choice, r["top"], dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def moe(h, W, p, f):
    r = f["router"]
    idx, wts = route(h, W, p, f)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t].tolist(), wts[t]):
            if e >= r["experts"]:
                y[t] += w * h[t]
            else:
                y[t] += w * expert(h[t:t + 1], W, f"{p}e{e}.", f["expert"]["limit"])[0]
    return y


# ------------------------------------------------------------------------------------------ the model
def mixer(h, W, p, L, eps):
    if L["type"] in ("attention", "attention_2"):
        return attention(h, W, p, L["mixer"], eps, L["type"])
    if L["type"] == "retention":
        return retention(h, W, p, L["mixer"], eps)
    raise ValueError(L["type"])


def forward(cfg, weights, tokens, after_layer=None):
    """Logits [S, vocab] of one sequence.  ``after_layer(i, x)`` sees the residual stream after every layer."""
    W = {k: v.to(F64) if v.is_floating_point() else v for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + mixer(rms_norm(x, eps) * W[p + "norm1"], W, p + "mix.", L, eps)
        if L.get("mlp") is not None:
            x = x + moe(rms_norm(x, eps) * W[p + "norm2"], W, p + "mlp.", L["mlp"])
        if after_layer is not None:
            after_layer(i, x)
    logits = (rms_norm(x, eps) * W["final.norm"]) @ W["head"].T
    cap = cfg.get("logit_softcap")
    return logits if not cap else cap * torch.tanh(logits / cap)
