"""The Vikarax decoder, plainly: float64, whole sequences, no cache, no state
carried between calls, one function per mechanism. It takes a decoded
config.json document and a dict of tensors by their file names, and shares no
code with `foundry_b200`. `state_space_stepwise` walks a sequence token by
token with an explicit state and guards the whole-sequence form
(tests/test_vikarax_cpu.py).

Notation: T tokens, W width, H heads, G key/value heads (or groups), d key
size, e value size, N state rows a head.
"""
import math

import torch

F = torch.float64


def layer_norm(x, w, b, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w + b


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0.0)


def rotate_half(x, positions, dims, base):
    """x [T, heads, d]: element i < dims/2 of a head turns with element i + dims/2 by
    the angle position * base^(-2i/dims); elements from `dims` on pass unchanged."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.pow(torch.tensor(base, dtype=F), -2.0 * torch.arange(half, dtype=F) / dims)
    angle = torch.as_tensor(positions, dtype=F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], -1)


def chunk_visible(i, j, size):
    """Whether the query at position i sees the key at position j."""
    return j <= i and (size is None or i // size == j // size)


def sigmoid_attention(m, w, p, h, eps):
    """The left mixer. m: its config entry; tensors `p.q|k|v|g|o`, `p.q.norm`,
    `p.k.norm`, `p.pb`; h [T, W] from position 0 on."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {}
    size = (m.get("mask") or {}).get("size")
    pos = list(range(T))
    q = rms_unit((h @ w[f"{p}.q"].T).view(T, H, d), eps) * w[f"{p}.q.norm"]
    k = rms_unit((h @ w[f"{p}.k"].T).view(T, G, d), eps) * w[f"{p}.k.norm"]
    q = rotate_half(q, pos, rot.get("dims", 0), rot.get("base", 10000.0))
    k = rotate_half(k, pos, rot.get("dims", 0), rot.get("base", 10000.0))
    v = rms_unit((h @ w[f"{p}.v"].T).view(T, G, e), eps)
    see = torch.tensor([[chunk_visible(i, j, size) for j in range(T)] for i in range(T)])
    gate = sigmoid(h @ w[f"{p}.g"].T)  # [T, H]
    heads = []
    for a in range(H):
        g = a // (H // G)
        score = (q[:, a] @ k[:, g].T) * m["scale"] + w[f"{p}.pb"][a]
        weight = torch.where(see, sigmoid(score), torch.zeros((), dtype=F))
        heads.append((weight @ v[:, g]) * gate[:, a:a + 1])
    return torch.cat(heads, -1) @ w[f"{p}.o"].T


def causal_conv_bias(x, taps_w, bias):
    """y[t, c] = sum_a taps_w[c, a] x[t - (taps - 1 - a), c] + bias[c], zeros before the start."""
    T, taps = x.shape[0], taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F), x], 0)
    return sum(padded[a:a + T] * taps_w[:, a] for a in range(taps)) + bias


def _state_space_inputs(m, w, p, h):
    H, e, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * e
    rows = h @ w[f"{p}.in"].T
    z, xbc, dt = rows[:, :inner], rows[:, inner:2 * inner + 2 * G * N], rows[:, 2 * inner + 2 * G * N:]
    return z, xbc, softplus(dt + w[f"{p}.dt_bias"])


def _state_space_output(m, w, p, y, z, eps):
    T, parts = y.shape[0], m.get("norm_groups", 1)
    y = y * silu(z)
    y = rms_unit(y.view(T, parts, -1), eps).reshape(T, -1) * w[f"{p}.norm"]
    return y @ w[f"{p}.o"].T


def state_space(m, w, p, h, eps):
    """The right mixer, in the attention-like form: the output at i is the sum over j <= i
    of (C_i . B_j) * (product of the decays after j up to i) * dt_j * x_j, plus D x_i."""
    T = h.shape[0]
    H, e, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * e
    z, xbc, dt = _state_space_inputs(m, w, p, h)
    xbc = silu(causal_conv_bias(xbc, w[f"{p}.conv"], w[f"{p}.conv.b"]))
    x = xbc[:, :inner].view(T, H, e)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    log_decay = -torch.exp(w[f"{p}.A_log"]) * dt  # [T, H]
    total = torch.cumsum(log_decay, 0)
    lower = torch.tril(torch.ones(T, T, dtype=torch.bool))
    heads = []
    for a in range(H):
        g = a // (H // G)
        between = torch.where(lower, total[:, a][:, None] - total[:, a][None, :],
                              torch.full((), -math.inf, dtype=F))
        weight = (C[:, g] @ B[:, g].T) * torch.exp(between) * dt[:, a][None, :]
        heads.append(weight @ x[:, a] + w[f"{p}.D"][a] * x[:, a])
    return _state_space_output(m, w, p, torch.cat(heads, -1), z, eps)


def state_space_stepwise(m, w, p, h, eps):
    """The same token by token: S <- exp(-exp(A_log) dt) S + dt B x^T; y = S^T C + D x, with
    the convolution's last inputs carried along."""
    T = h.shape[0]
    H, e, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, taps = H * e, w[f"{p}.conv"].shape[1]
    z, xbc, dt = _state_space_inputs(m, w, p, h)
    S = torch.zeros(H, N, e, dtype=F)
    tail = torch.zeros(taps - 1, xbc.shape[1], dtype=F)
    out = torch.zeros(T, inner, dtype=F)
    for t in range(T):
        window = torch.cat([tail, xbc[t:t + 1]], 0)
        tail = window[1:]
        row = silu((window * w[f"{p}.conv"].T).sum(0) + w[f"{p}.conv.b"])
        x, B, C = row[:inner].view(H, e), row[inner:inner + G * N].view(G, N), \
            row[inner + G * N:].view(G, N)
        for a in range(H):
            g = a // (H // G)
            S[a] = torch.exp(-torch.exp(w[f"{p}.A_log"][a]) * dt[t, a]) * S[a] + \
                dt[t, a] * torch.outer(B[g], x[a])
            out[t, a * e:(a + 1) * e] = S[a].T @ C[g] + w[f"{p}.D"][a] * x[a]
    return _state_space_output(m, w, p, out, z, eps)


def parallel_mixer(m, w, p, h, eps):
    return m.get("left_scale", 1.0) * sigmoid_attention(m["left"], w, f"{p}.left", h, eps) + \
        m.get("right_scale", 1.0) * state_space(m["right"], w, f"{p}.right", h, eps)


def dense_feed_forward(w, p, h):
    return torch.relu(h @ w[f"{p}.up"].T) ** 2 @ w[f"{p}.down"].T


def gated_expert(w, p, h):
    return (silu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def route(mlp, scores):
    """The chosen experts of one token, in falling order of their scores [E]."""
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = E // groups["count"]
    of_group = []
    for g in range(groups["count"]):
        best = sorted(scores[g * per:(g + 1) * per].tolist(), reverse=True)
        of_group.append(sum(best[:2]))
    kept = sorted(range(groups["count"]), key=lambda g: (-of_group[g], g))[:groups["keep"]]
    allowed = [x for x in range(E) if x // per in kept]
    return sorted(allowed, key=lambda x: (-float(scores[x]), x))[:top]


def route_margin(mlp, scores):
    """How far one token's choice is from another one: the gap between the last kept
    group and the first dropped one, and between the last chosen expert and the first
    allowed one that is not chosen; the smaller of the two (inf where nothing is dropped)."""
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = E // groups["count"]
    of_group = [sum(sorted(scores[g * per:(g + 1) * per].tolist(), reverse=True)[:2])
                for g in range(groups["count"])]
    order = sorted(range(groups["count"]), key=lambda g: (-of_group[g], g))
    keep = groups["keep"]
    gap = of_group[order[keep - 1]] - of_group[order[keep]] if keep < len(order) else float("inf")
    allowed = sorted((float(scores[x]) for x in range(E) if x // per in order[:keep]), reverse=True)
    if top < len(allowed):
        gap = min(gap, allowed[top - 1] - allowed[top])
    return gap


def routed_experts(mlp, w, p, h, margins=None):
    scores = sigmoid(h @ w[f"{p}.router"].T)
    if margins is not None:
        margins.append([route_margin(mlp, scores[t]) for t in range(h.shape[0])])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for x in route(mlp, scores[t]):
            out[t] += scores[t, x] * gated_expert(w, f"{p}.e{x}", h[t:t + 1])[0]
    if mlp.get("shared"):
        out = out + gated_expert(w, f"{p}.shared", h)
    return out


def layer(cfg, w, i, x, margins=None):
    """The result of layer i (before the weighted sum over the streams)."""
    entry, p, eps = cfg["layers"][i], f"l{i}", cfg["norm"]["eps"]
    norm = lambda name, t: layer_norm(t, w[f"{p}.{name}"], w[f"{p}.{name}.b"], eps)
    x = x + norm("norm1b", parallel_mixer(entry["mixer"], w, f"{p}.mix", norm("norm1", x), eps))
    mlp = entry["mlp"]
    if mlp is not None:
        h = norm("norm2", x)
        y = dense_feed_forward(w, f"{p}.mlp", h) if mlp["kind"] == "dense" else \
            routed_experts(mlp, w, f"{p}.mlp", h, margins)
        x = x + norm("norm2b", y)
    return x


def depth_average(kept, weights):
    return sum(weights[j] * kept[j] for j in range(len(kept)))


def forward(cfg, w, tokens, streams=None, margins=None):
    """Logits [T, vocab] of a whole sequence; `streams` collects what leaves each layer,
    `margins` the routers' margins (`route_margin`), a list per routed layer."""
    x = w["embed"][torch.as_tensor(tokens)]
    kept = [x]
    for i in range(len(cfg["layers"])):
        kept.append(layer(cfg, w, i, x, margins))
        x = depth_average(kept, w[f"l{i}.dwa"])
        if streams is not None:
            streams.append(x)
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], cfg["norm"]["eps"])
    logits = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy_generate(cfg, w, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(torch.argmax(forward(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]
