"""The Kutepel decoder, plainly: float64, whole sequences, no cache, one function
per mechanism. It takes a decoded config.json document and a dict of tensors by
their file names, and shares no code with `foundry_b200`. The `*_stepwise`
variants walk a sequence token by token over explicit key lists and guard the
whole-sequence forms (tests/test_kutepel_cpu.py).

Notation: T tokens, W width, H heads, G key heads, d key size, e value size,
r latent size, c rotated size, p a token's position, m the residual constant.
"""
import math

import torch

F = torch.float64
WEIGHT_SUM_FLOOR = 1e-20  # joins the sum of the chosen experts' scores


def layer_norm(x, w, eps):
    mean = x.mean(-1, keepdim=True)
    dev = x - mean
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(x):
    return x / (1.0 + torch.exp(-x))


# ------------------------------------------------------------------- rotation
def frequencies(rot):
    """f_i = base^(-2i / dims), i < dims / 2; with `scaling`, long wavelengths are
    slowed by `factor`, short ones kept, and those between blended."""
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    s = rot.get("scaling")
    if not s:
        return f
    factor, low, high, original = s["factor"], s["low"], s["high"], s["original"]
    out = f.clone()
    for i in range(f.numel()):
        wavelength = 2.0 * math.pi / f[i].item()
        if wavelength < original / high:
            continue
        if wavelength > original / low:
            out[i] = f[i] / factor
        else:
            blend = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - blend) * f[i] / factor + blend * f[i]
    return out


def rotate(x, positions, freq):
    """x [T, ..., n]: elements (2i, 2i + 1), i < len(freq), turned by p f_i; the rest kept."""
    n = 2 * freq.numel()
    angle = positions.to(F)[:, None] * freq[None, :]
    while angle.dim() < x.dim():
        angle = angle.unsqueeze(1)
    cos, sin = torch.cos(angle), torch.sin(angle)
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = u * cos - v * sin
    out[..., 1:n:2] = v * cos + u * sin
    return out


# ------------------------------------------------------------------ attention
def attention_keys_values(m, w, p, h, positions):
    """What a layer keeps of its input: keys (rotated) [T, G, d] and values [T, G, e]."""
    T = h.shape[0]
    G, d, e = m["kv_heads"], m["dim"], m["vdim"]
    k = rotate((h @ w[p + ".k"].T).view(T, G, d), positions, frequencies(m["rot"]))
    return k, (h @ w[p + ".v"].T).view(T, G, e)


def softmax_with_sink(scores, sink):
    """scores [T, T'] already masked with -inf; `sink` joins the denominator once
    (None: the ordinary softmax)."""
    top = scores.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, torch.full_like(top, float(sink)))
    weights = torch.exp(scores - top)
    total = weights.sum(-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink - top)
    return weights / total


def causal_mask(T):
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


def attention(m, w, p, h, positions, kv=None):
    """Grouped heads with rotated queries and keys and a learned sink per head. `kv`:
    keys and values of another layer (a layer with `kv_from`)."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate((h @ w[p + ".q"].T).view(T, H, d), positions, frequencies(m["rot"]))
    k, v = attention_keys_values(m, w, p, h, positions) if kv is None else kv
    seen = causal_mask(T)
    out = torch.zeros(T, H, e, dtype=F)
    for a in range(H):
        g = a // (H // G)
        scores = (q[:, a] @ k[:, g].T) * m["scale"]
        scores = scores.masked_fill(~seen, -math.inf)
        out[:, a] = softmax_with_sink(scores, w[p + ".sink"][a]) @ v[:, g]
    return out.reshape(T, H * e) @ w[p + ".o"].T


def attention_stepwise(m, w, p, h, positions, kv=None):
    """The same, token by token over explicit key and value lists."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    freq = frequencies(m["rot"])
    rows = []
    keys, values = [], []
    for t in range(T):
        x, pos = h[t:t + 1], positions[t:t + 1]
        q = rotate((x @ w[p + ".q"].T).view(1, H, d), pos, freq)[0]
        if kv is None:
            keys.append(rotate((x @ w[p + ".k"].T).view(1, G, d), pos, freq)[0])
            values.append((x @ w[p + ".v"].T).view(G, e))
            K, V = torch.stack(keys), torch.stack(values)
        else:
            K, V = kv[0][:t + 1], kv[1][:t + 1]
        o = torch.zeros(H, e, dtype=F)
        for a in range(H):
            g = a // (H // G)
            s = (K[:, g] @ q[a]) * m["scale"]
            weights = torch.exp(s)
            o[a] = (weights[:, None] * V[:, g]).sum(0) / (weights.sum() + torch.exp(w[p + ".sink"][a]))
        rows.append(o.reshape(1, H * e) @ w[p + ".o"].T)
    return torch.cat(rows, 0)


# ----------------------------------------------------------- latent attention
def latent_rows(m, w, p, h, positions, eps):
    """What a layer keeps of its input: the latent [T, r] and one rotated key part [T, c]."""
    r = m["kv_rank"]
    down = h @ w[p + ".dkv"].T
    latent = rms_norm(down[:, :r], w[p + ".dkv.norm"], eps)
    return latent, rotate(down[:, r:], positions, frequencies(m["rot"]))


def latent_attention(m, w, p, h, positions, eps):
    T = h.shape[0]
    H, d, c, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + ".q"].T).view(T, H, d + c)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], positions, frequencies(m["rot"]))
    latent, k_rot = latent_rows(m, w, p, h, positions, eps)
    k_plain = (latent @ w[p + ".uk"].T).view(T, H, d)
    v = (latent @ w[p + ".uv"].T).view(T, H, e)
    seen = causal_mask(T)
    out = torch.zeros(T, H, e, dtype=F)
    for a in range(H):
        scores = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        scores = scores.masked_fill(~seen, -math.inf)
        out[:, a] = softmax_with_sink(scores, None) @ v[:, a]
    gate = torch.sigmoid(h @ w[p + ".g"].T)
    return (out.reshape(T, H * e) * gate) @ w[p + ".o"].T


def latent_attention_stepwise(m, w, p, h, positions, eps):
    """Token by token over the kept rows only, with the expansions folded into the
    query and the output: q_plain . (W_uk l) = (W_uk^T q_plain) . l."""
    T = h.shape[0]
    H, d, c, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    freq = frequencies(m["rot"])
    uk = w[p + ".uk"].view(H, d, r)
    uv = w[p + ".uv"].view(H, e, r)
    kept = []
    rows = []
    for t in range(T):
        x, pos = h[t:t + 1], positions[t:t + 1]
        latent, k_rot = latent_rows(m, w, p, x, pos, eps)
        kept.append(torch.cat([latent[0], k_rot[0]]))
        K = torch.stack(kept)
        q = (x @ w[p + ".q"].T).view(1, H, d + c)
        q_rot = rotate(q[..., d:], pos, freq)[0]
        o = torch.zeros(H, e, dtype=F)
        for a in range(H):
            wide = torch.cat([uk[a].T @ q[0, a, :d], q_rot[a]])
            s = (K @ wide) * m["scale"]
            weights = torch.softmax(s, 0)
            o[a] = uv[a] @ (weights[:, None] * K[:, :r]).sum(0)
        gate = torch.sigmoid(x @ w[p + ".g"].T)
        rows.append((o.reshape(1, H * e) * gate) @ w[p + ".o"].T)
    return torch.cat(rows, 0)


# -------------------------------------------------------------- routed experts
def route(router, z, correction):
    """z [T, E] router logits. Returns chosen [T, top] and weights [T, top]."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    scores = torch.sigmoid(z)
    choice = scores + correction
    size = E // count
    chosen_all, weights_all = [], []
    for t in range(z.shape[0]):
        ranks = [sum(sorted(choice[t, g * size:(g + 1) * size].tolist(), reverse=True)[:2])
                 for g in range(count)]
        best = sorted(range(count), key=lambda g: (-ranks[g], g))[:keep]
        allowed = [i for i in range(E) if i // size in best]
        chosen = sorted(allowed, key=lambda i: (-choice[t, i].item(), i))[:top]
        s = scores[t, chosen]
        chosen_all.append(chosen)
        weights_all.append(s / (s.sum() + WEIGHT_SUM_FLOOR) * router["scale"])
    return torch.tensor(chosen_all), torch.stack(weights_all)


def expert(w, p, h):
    return (silu(h @ w[p + ".gate"].T) * (h @ w[p + ".up"].T)) @ w[p + ".down"].T


def routed_experts(mlp, w, p, h):
    z = h @ w[p + ".router"].T
    chosen, weights = route(mlp["router"], z, w[p + ".correction"])
    out = torch.zeros(h.shape[0], w[p + ".e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for j, i in enumerate(chosen[t].tolist()):
            out[t] += weights[t, j] * expert(w, f"{p}.e{i}", h[t:t + 1])[0]
    return out


def router_margins(mlp, w, p, h):
    """Per token, the smallest gap that a change of the scores would have to bridge to
    change the choice: between the last chosen and the first left out, and between the
    last kept and the first dropped group."""
    router = mlp["router"]
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    size = E // count
    choice = torch.sigmoid(h @ w[p + ".router"].T) + w[p + ".correction"]
    out = []
    for t in range(h.shape[0]):
        ranks = [sum(sorted(choice[t, g * size:(g + 1) * size].tolist(), reverse=True)[:2])
                 for g in range(count)]
        order = sorted(range(count), key=lambda g: (-ranks[g], g))
        gap = math.inf if keep == count else ranks[order[keep - 1]] - ranks[order[keep]]
        allowed = sorted((choice[t, i].item() for i in range(E) if i // size in order[:keep]),
                         reverse=True)
        if top < len(allowed):
            gap = min(gap, allowed[top - 1] - allowed[top])
        out.append(gap)
    return torch.tensor(out, dtype=F)


# ------------------------------------------------------------------ the model
def layer_update(cfg, w, i, x, positions, kept):
    """x <- x + m (mixer(h) + ff(h)), h = LN(x). `kept[j]` holds layer j's keys and values."""
    layer = cfg["layers"][i]
    m, eps, p = layer["mixer"], cfg["norm"]["eps"], f"l{i}"
    h = layer_norm(x, w[p + ".norm1"], eps)
    if layer["type"] == "attention":
        source = m.get("kv_from")
        if source is None:
            kept[i] = attention_keys_values(m, w, p + ".mix", h, positions)
            y = attention(m, w, p + ".mix", h, positions)
        else:
            y = attention(m, w, p + ".mix", h, positions, kv=kept[source])
    else:
        y = latent_attention(m, w, p + ".mix", h, positions, eps)
    if layer.get("mlp"):
        y = y + routed_experts(layer["mlp"], w, p + ".mlp", h)
    return x + cfg["residual_mult"] * y


def forward(cfg, weights, tokens, return_streams=False):
    """Logits [T, vocab] of one whole sequence from position 0."""
    w = {k: v.to(F) for k, v in weights.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(ids.numel())
    x = w["embed"][ids]
    kept, streams = {}, []
    for i in range(len(cfg["layers"])):
        x = layer_update(cfg, w, i, x, positions, kept)
        streams.append(x)
    logits = layer_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].T
    return (logits, torch.stack(streams)) if return_streams else logits
