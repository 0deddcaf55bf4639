"""A plain, slow implementation of the Sapatar decoder: one function per mechanism, whole sequences, no cache,
no kernels, token-by-token loops where the design is a recurrence.  It shares no code with the engine and is what
the engine's parts and models are compared with.  ``w`` is a dict of tensors by checkpoint name, ``cfg`` the
contents of config.json.  Everything runs in the type of the tensors handed in (float64 for a sharp comparison).
"""
import torch


# ---------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------
def rms(x, weight=None, eps=1e-6):
    """x / sqrt(mean(x^2) + eps) over the last axis, times ``weight`` where one is given."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(x):
    return x * torch.sigmoid(x)


def rotate_half_layout(x, positions, dims, base):
    """x [T, H, D]: value i of a head is paired with value i + dims/2 (i < dims/2) and the pair is turned by
    the angle position * base**(-2i/dims); values from ``dims`` on stay."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.tensor(float(base), dtype=x.dtype) ** (-2.0 * i / dims)
    angle = positions.to(x.dtype)[:, None, None] * freq
    cos, sin = torch.cos(angle), torch.sin(angle)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------
# token mixing, each on tensors that are already projected
# ---------------------------------------------------------------------------
def window_softmax_attention(q, k, v, scale, window):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; query head h reads key/value head h // (H / G); token t sees the
    tokens j with 0 <= t - j < window (all earlier ones when window is None)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        t = torch.arange(T)
        seen = (t[:, None] >= t[None, :])
        if window is not None:
            seen &= (t[:, None] - t[None, :]) < window
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def retention_recurrence(q, k, v, decay):
    """q, k [T, H, D], v [T, H, Dv], decay [H]:  S <- decay_h S + k v^T, then o = S^T q (the new state)."""
    T, H, D = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        S = torch.zeros(D, v.shape[2], dtype=q.dtype)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def wkv_recurrence(r, k, v, w, u):
    """r, k, v, w [T, H, D], u [H, D]:  o = (S + diag(u) k v^T)^T r with the old state, then
    S <- diag(w) S + k v^T."""
    T, H, D = r.shape
    out = torch.zeros(T, H, D, dtype=r.dtype)
    for h in range(H):
        S = torch.zeros(D, D, dtype=r.dtype)
        for t in range(T):
            kv = torch.outer(k[t, h], v[t, h])
            out[t, h] = (S + u[h][:, None] * kv).T @ r[t, h]
            S = w[t, h][:, None] * S + kv
    return out


def mlstm_recurrence(q, k, v, log_i, log_f):
    """q, k [T, H, D], v [T, H, Dv], log gates [T, H].  A running maximum m (0 before the first token) keeps
    the exponentials bounded:  m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise with k;
    o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)."""
    T, H, D = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        S = torch.zeros(D, v.shape[2], dtype=q.dtype)
        n = torch.zeros(D, dtype=q.dtype)
        m = torch.zeros((), dtype=q.dtype)
        for t in range(T):
            m_new = torch.maximum(log_f[t, h] + m, log_i[t, h])
            a, b = torch.exp(log_f[t, h] + m - m_new), torch.exp(log_i[t, h] - m_new)
            S = a * S + b * torch.outer(k[t, h], v[t, h])
            n = a * n + b * k[t, h]
            m = m_new
            out[t, h] = (S.T @ q[t, h]) / (torch.maximum((n @ q[t, h]).abs(), torch.exp(-m)) + 1e-6)
    return out


# ---------------------------------------------------------------------------
# mixers: projections around the above
# ---------------------------------------------------------------------------
def mixer_wkv(h, w, p, m, eps):
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]])
    mixed = {s: h + (prev - h) * w[f"{p}.mu.{s}"] for s in "rkvgw"}
    r = (mixed["r"] @ w[f"{p}.r"].T).view(T, H, D)
    k = (mixed["k"] @ w[f"{p}.k"].T).view(T, H, D)
    v = (mixed["v"] @ w[f"{p}.v"].T).view(T, H, D)
    gate = silu(mixed["g"] @ w[f"{p}.g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mixed["w"] @ w[f"{p}.w1"].T) @ w[f"{p}.w2"].T + w[f"{p}.w0"])).view(T, H, D)
    o = rms(wkv_recurrence(r, k, v, decay, w[f"{p}.u"]), None, eps).reshape(T, H * D)
    return (o * w[f"{p}.norm"] * gate) @ w[f"{p}.o"].T


def mixer_retention(h, w, p, m, eps, positions):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = rotate_half_layout((h @ w[f"{p}.q"].T).view(T, H, D), positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half_layout((h @ w[f"{p}.k"].T).view(T, H, D), positions, m["rot"]["dims"], m["rot"]["base"]) * D ** -0.5
    v = (h @ w[f"{p}.v"].T).view(T, H, Dv)
    o = rms(retention_recurrence(q, k, v, torch.tensor(m["decay"], dtype=h.dtype)), None, eps).reshape(T, H * Dv)
    return (o * silu(h @ w[f"{p}.g"].T)) @ w[f"{p}.o"].T


def mixer_softmax(h, w, p, m, positions):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[f"{p}.q"].T + w[f"{p}.q.b"]).view(T, H, D)
    k = (h @ w[f"{p}.k"].T + w[f"{p}.k.b"]).view(T, G, D)
    v = (h @ w[f"{p}.v"].T + w[f"{p}.v.b"]).view(T, G, Dv)
    q = rotate_half_layout(q, positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half_layout(k, positions, m["rot"]["dims"], m["rot"]["base"])
    window = m["mask"]["size"] if m.get("mask") else None
    return window_softmax_attention(q, k, v, m["scale"], window).reshape(T, H * Dv) @ w[f"{p}.o"].T


def mixer_mlstm(h, w, p, m, eps):
    T = h.shape[0]
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[f"{p}.q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[f"{p}.k"].T).view(T, H, D)
    v = (h @ w[f"{p}.v"].T).view(T, H, Dv)
    log_i = cap * torch.tanh((h @ w[f"{p}.i"].T + w[f"{p}.i.b"]) / cap)
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[f"{p}.f"].T + w[f"{p}.f.b"]) / cap))
    o = rms(mlstm_recurrence(q, k, v, log_i, log_f), None, eps).reshape(T, H * Dv)
    return (o * w[f"{p}.norm"] * torch.sigmoid(h @ w[f"{p}.g"].T)) @ w[f"{p}.o"].T


def mixer(kind, h, w, p, m, eps, positions):
    if kind == "wkv":
        return mixer_wkv(h, w, p, m, eps)
    if kind == "retention":
        return mixer_retention(h, w, p, m, eps, positions)
    if kind == "parallel":
        return (m["left_scale"] * mixer_softmax(h, w, f"{p}.left", m["left"], positions)
                + m["right_scale"] * mixer_mlstm(h, w, f"{p}.right", m["right"], eps))
    raise ValueError(kind)


# ---------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------
def gated_expert(h, w, p):
    return (silu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def route(h, w, p, top):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over those alone."""
    z = h @ w[f"{p}.router"].T + w[f"{p}.router.b"]
    best, chosen = torch.topk(z, top, dim=-1)
    return chosen, torch.softmax(best, dim=-1)


def feed_forward_moe(h, w, p, mlp):
    chosen, weight = route(h, w, p, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(chosen[t].tolist(), weight[t]):
            out[t] += c * gated_expert(h[t], w, f"{p}.e{e}")
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[f"{p}.shared.sg"].T) * gated_expert(h, w, f"{p}.shared")
    return out


# ---------------------------------------------------------------------------
# layers and the model
# ---------------------------------------------------------------------------
def hyper_read(streams, w, p):
    """streams [s, T, width] -> the sub-layer's input, a weighted sum of the copies."""
    return torch.einsum("s,stc->tc", w[f"{p}.in"], streams)


def hyper_write(streams, y, w, p):
    """All copies at once from the old ones: x_t <- sum_s mix[s, t] x_s + out[t] y."""
    return torch.einsum("st,snc->tnc", w[f"{p}.mix"], streams) + w[f"{p}.out"][:, None, None] * y[None]


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from its first token; with ``return_layers`` also the residual rows
    (the sum of the copies) after every layer run."""
    eps = cfg["norm"]["eps"]
    dtype = w["embed"].dtype
    positions = torch.arange(len(tokens))
    x = w["embed"][torch.tensor(tokens)]
    copies = cfg.get("streams")
    streams = torch.stack([x] * copies) if copies else None
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}" if layer.get("weights_of") is not None else f"l{i}"
        subs = [(1, lambda h: mixer(layer["type"], h, w, f"{p}.mix", layer["mixer"], eps, positions))]
        if layer.get("mlp") is not None:
            subs.append((2, lambda h: feed_forward_moe(h, w, f"{p}.mlp", layer["mlp"])))
        for nr, f in subs:
            if copies:
                y = f(rms(hyper_read(streams, w, f"{p}.hc{nr}"), w[f"{p}.norm{nr}"], eps))
                streams = hyper_write(streams, y, w, f"{p}.hc{nr}")
            else:
                x = x + f(rms(x, w[f"{p}.norm{nr}"], eps))
        after.append(streams.sum(0) if copies else x)
    x = after[-1] if cfg["layers"] else x
    logits = rms(x, w["final.norm"], eps) @ w["head"].T
    assert logits.dtype == dtype
    return (logits, torch.stack(after)) if return_layers else logits


# ---------------------------------------------------------------------------
# model folders
# ---------------------------------------------------------------------------
def read_folder(folder, dtype=torch.float32):
    """config.json and every tensor of model.safetensors, read with nothing but struct-like slicing and torch."""
    import json
    from pathlib import Path
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    n = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32}
    weights = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=kinds[meta["dtype"]]).view(meta["shape"])
        weights[name] = t.to(dtype) if t.is_floating_point() else t
    return config, weights


def logits_of(folder, tokens, dtype=torch.float64) -> torch.Tensor:
    config, weights = read_folder(folder, dtype)
    return forward(config, weights, tokens).float()


def greedy(folder, prompt, steps):
    """Greedy continuation, the slow way: the whole sequence again for every token (lowest index at a tie)."""
    config, weights = read_folder(folder, torch.float64)
    tokens, out = list(prompt), []
    for _ in range(steps):
        nxt = int(torch.argmax(forward(config, weights, tokens)[-1]))
        out.append(nxt)
        tokens.append(nxt)
    return out
