"""A plain, slow implementation of the Linurax decoder, written from its equations: the oracle
of the tests.  One function per mechanism, whole sequences at once, no cache, no batching,
nothing shared with the engine.  Everything runs on the CPU in the type of the weights it is
given (float32, or float64 for a sharper oracle).

The design, in this file's notation (x: residual rows [T, width]; W stored [out, in]):

    x      = E[token] * embedding_scale
    layer:   x += rms(mixer(x)) * n1          (the norm sits on the sublayer's OUTPUT; the sublayer reads x itself)
             x += rms(ff(x)) * n2             (only if the layer has a feed-forward)
    rms(y) = y / sqrt(mean(y^2) + eps)
    logits = E @ (rms(x) * n_final)           (E itself, not scaled)

    mixer "attention" (H query heads, G key/value heads, head size D):
        q = Wq x, k = Wk x, v = k              (the values are the keys as projected)
        q = rms(q) * nq, k = rms(k) * nk       (each over the WHOLE projection, all heads at once)
        q, k rotated on the first R dims of every head, pair (2i, 2i+1), angle p * base^(-2i/R)
        s[h] = scale * q_h . k_{h // (H/G)}    for keys j <= i
        s[h] <- sum_g Talk[h, g] s[g]
        w[h] = sigmoid(s[h] + pb[h])           (no normalisation over keys)
        o_h  = sum_j w[h][i, j] v_{h // (H/G)}[j]
        out  = Wo (concat(o) * sigmoid(Wg x))

    mixer "mingru" (state of `width` values per sequence, zero at the start):
        z = sigmoid(Wz x + bz), u = Wx x + bx, c = u + 1/2 if u >= 0 else sigmoid(u)
        S_t = (1 - z_t) S_{t-1} + z_t c_t
        out = Wo (S_t * silu(Wg x))

    feed-forward: Wdown (silu(Wgate x) * (Wup x))
"""
from __future__ import annotations

import json
from pathlib import Path

import torch


def rms(y: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps) * weight


def rotate_interleaved(t: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """t: [T, heads, D].  The first ``dims`` values of each head are rotated pair-wise, (2i, 2i+1)."""
    out = t.clone()
    i = torch.arange(dims // 2, dtype=t.dtype)
    freq = torch.tensor(base, dtype=t.dtype) ** (-2.0 * i / dims)
    ang = positions.to(t.dtype)[:, None] * freq[None, :]                 # [T, dims/2]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = t[..., 0:dims:2], t[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def sigmoid_attention(x: torch.Tensor, w: dict, p: dict, eps: float, start: int = 0, window: int | None = None) -> torch.Tensor:
    """x: [T, width] rows of one sequence whose first row sits at position ``start`` (always 0 here).
    ``window`` (not part of the design; the engine's mixer has it as an option): only keys j > i - window."""
    T = x.shape[0]
    H, G, D = p["heads"], p["kv_heads"], p["dim"]
    q = x @ w["q"].T
    k = x @ w["k"].T
    v = k.view(T, G, D)
    q = rms(q, w["q.norm"], eps).view(T, H, D)
    k = rms(k, w["k.norm"], eps).view(T, G, D)
    pos = torch.arange(start, start + T)
    q = rotate_interleaved(q, pos, p["rot"]["dims"], p["rot"]["base"])
    k = rotate_interleaved(k, pos, p["rot"]["dims"], p["rot"]["base"])
    group = H // G
    kh = k.repeat_interleave(group, dim=1)                               # query head h reads kv head h // group
    vh = v.repeat_interleave(group, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kh) * p["scale"]                 # [H, T, T]
    s = torch.einsum("hg,gij->hij", w["talk"], s)
    weight = torch.sigmoid(s + w["pb"][:, None, None])
    visible = torch.ones(T, T, dtype=torch.bool).tril()
    if window is not None:
        visible = visible & ~torch.ones(T, T, dtype=torch.bool).tril(-window)
    weight = weight * visible
    o = torch.einsum("hij,jhd->ihd", weight, vh).reshape(T, H * D)
    o = o * torch.sigmoid(x @ w["g"].T)
    return o @ w["o"].T


def mingru(x: torch.Tensor, w: dict) -> torch.Tensor:
    T = x.shape[0]
    z = torch.sigmoid(x @ w["z"].T + w["z.b"])
    u = x @ w["x"].T + w["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = x @ w["g"].T
    gate = gate * torch.sigmoid(gate)
    S = torch.zeros(z.shape[1], dtype=x.dtype)
    rows = []
    for t in range(T):
        S = (1 - z[t]) * S + z[t] * cand[t]
        rows.append(S * gate[t])
    return torch.stack(rows) @ w["o"].T


def dense_ff(x: torch.Tensor, w: dict) -> torch.Tensor:
    g = x @ w["gate"].T
    return ((g * torch.sigmoid(g)) * (x @ w["up"].T)) @ w["down"].T


def sub(weights: dict, prefix: str) -> dict:
    """The tensors below ``prefix.`` with that prefix taken off."""
    return {k[len(prefix) + 1:]: v for k, v in weights.items() if k.startswith(prefix + ".")}


def forward(config: dict, weights: dict, tokens: list[int], keep_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and, on request, the residual rows after every layer)."""
    eps = config["norm"]["eps"]
    E = weights["embed"]
    x = E[torch.tensor(tokens)] * config["embedding"]["scale"]
    after = []
    for i, layer in enumerate(config["layers"]):
        name = f"l{i}"
        if layer["type"] == "attention":
            y = sigmoid_attention(x, sub(weights, f"{name}.mix"), layer["mixer"], eps)
        elif layer["type"] == "mingru":
            y = mingru(x, sub(weights, f"{name}.mix"))
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        x = x + rms(y, weights[f"{name}.norm1"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")
            x = x + rms(dense_ff(x, sub(weights, f"{name}.mlp")), weights[f"{name}.norm2"], eps)
        after.append(x)
    logits = rms(x, weights["final.norm"], eps) @ E.T
    return (logits, torch.stack(after)) if keep_layers else logits


def read_folder(folder, dtype=torch.float32):
    """config.json and every tensor of model.safetensors, read with nothing but struct and torch."""
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


def logits_of(folder, tokens, dtype=torch.float32) -> torch.Tensor:
    config, weights = read_folder(folder, dtype)
    return forward(config, weights, tokens)


def greedy(folder, prompt: list[int], steps: int) -> list[int]:
    """Greedy continuation, the slow way: the whole sequence again for every token (lowest index at a tie)."""
    config, weights = read_folder(folder)
    tokens, out = list(prompt), []
    for _ in range(steps):
        nxt = int(torch.argmax(forward(config, weights, tokens)[-1]))
        out.append(nxt)
        tokens.append(nxt)
    return out

