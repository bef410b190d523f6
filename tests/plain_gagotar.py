"""A plain, slow Gagotar: whole sequences, no cache, one function per mechanism, CPU torch.

Gagotar is a pre-norm decoder. A layer's mixer runs two mixers side by side on the same
normed input: a softmax attention (grouped keys, biases, a norm over the whole query and key
projections, partial rotary positions with scaled frequencies, a number per head and a
mixing of the heads' scores before the softmax, keys visible only inside the query's own
chunk of positions, one output gate per head) and a gated linear attention with a decay per
key channel. Each side's result is normed over the model width and the two are averaged. The
feed-forward is a mixture of experts with clamped gated units. Both halves of a layer are
scaled element by element before they join the residual stream.

This file restates the formulas as whole-sequence sums or token by token and shares no code
with ``ayaka_b200``: it reads a checkpoint-named state dict and the plain dict of
``config.json``. Every function computes in the dtype of its inputs; tests pass float64.

Notation: ``x`` residual stream ``[T, width]``, ``h`` a normed input, ``t``/``s`` query and key
positions (from 0), ``H`` query heads, ``G`` key/value heads.
"""

from __future__ import annotations

import math

import torch

# ---------------------------------------------------------------------------------------------
# small pieces


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension (eps under the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def weighted_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * weight


def linear(x: torch.Tensor, weight_out_in: torch.Tensor,
           bias: torch.Tensor | None = None) -> torch.Tensor:
    y = x @ weight_out_in.T
    return y if bias is None else y + bias


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def scaled_frequencies(dims: int, base: float, scaling: dict | None) -> list[float]:
    """f_i = base^(-2i/dims) for the dims/2 pairs; with ``scaling`` (factor, low, high,
    original) a pair whose wavelength 2 pi / f is above original/low turns ``factor`` times
    slower, one below original/high is kept, and between the two the slowed and the kept
    frequency are blended linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high = scaling["factor"], scaling["low"], scaling["high"]
            original = scaling["original"]
            wavelength = 2.0 * math.pi / f
            if wavelength > original / low:
                f = f / factor
            elif wavelength >= original / high:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_halves(v: torch.Tensor, positions: torch.Tensor, freq: list[float]) -> torch.Tensor:
    """Rotary encoding on the first ``2 len(freq)`` entries of the last dimension: entry i is
    paired with entry i + len(freq) and the pair turned by position * freq[i]; the rest of
    the vector passes. ``v`` is [T, heads, D]; ``positions`` [T]."""
    half = len(freq)
    out = v.clone()
    if half == 0:
        return out
    angle = positions.to(v.dtype)[:, None] * torch.tensor(freq, dtype=v.dtype)[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = v[..., :half], v[..., half:2 * half]
    out[..., :half] = a * cos - b * sin
    out[..., half:2 * half] = b * cos + a * sin
    return out


def chunk_mask(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: key s is visible to query t when s <= t and both lie in the same block
    of ``size`` positions counted from 0."""
    t = torch.arange(T)
    return (t[None, :] <= t[:, None]) & ((t[None, :] // size) == (t[:, None] // size))


def mixed_head_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                         talk: torch.Tensor, temp: torch.Tensor, scale: float,
                         size: int) -> torch.Tensor:
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim] -> [T, H, vdim]. Head a's raw score is
    scale * temp[a] * (q_a . k_(a // (H/G))); every (t, s) pair's H scores are mixed by
    ``talk`` (score_h = sum_a talk[h, a] raw_a); softmax over the keys of t's own block of
    ``size`` positions up to t; head h sums the values of its own key/value head."""
    T, H, _ = q.shape
    per = H // k.shape[1]
    raw = torch.stack([q[:, a, :] @ k[:, a // per, :].T for a in range(H)])  # [H, T, T]
    raw = raw * scale * temp[:, None, None]
    score = torch.einsum("ha,ats->hts", talk, raw)
    score = score.masked_fill(~chunk_mask(T, size)[None], float("-inf"))
    weight = torch.softmax(score, dim=-1)
    return torch.stack([weight[h] @ v[:, h // per, :] for h in range(H)], dim=1)


def decayed_memory(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor,
                   tau: float, state: torch.Tensor | None = None
                   ) -> tuple[torch.Tensor, torch.Tensor]:
    """q, k, z [T, H, dim], v [T, H, vdim]. Token by token S <- diag(sigmoid(z)^(1/tau)) S +
    k v^T and out = S^T q; returns out [T, H, vdim] and the last S [H, dim, vdim]."""
    T, H, dim = q.shape
    decay = torch.sigmoid(z) ** (1.0 / tau)
    S = torch.zeros(H, dim, v.shape[2], dtype=q.dtype) if state is None else state.clone()
    out = torch.empty(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out, S


# ---------------------------------------------------------------------------------------------
# the two sides of the mixer


def softmax_side(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """The attention side. ``w`` holds this side's tensors without the prefix."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = linear(h, w["q"], w["q.b"])
    k = linear(h, w["k"], w["k.b"])
    v = linear(h, w["v"], w["v.b"]).reshape(T, G, vdim)
    # one norm over all heads' entries at once, then the split into heads
    q = weighted_norm(q, w["q.norm"], eps).reshape(T, H, dim)
    k = weighted_norm(k, w["k.norm"], eps).reshape(T, G, dim)
    rot = m["rot"]
    freq = scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    q, k = rotate_halves(q, positions, freq), rotate_halves(k, positions, freq)
    out = mixed_head_attention(q, k, v, w["talk"], w["temp"], m["scale"], m["mask"]["size"])
    gate = torch.sigmoid(linear(h, w["g"]))  # [T, H]: one number per head
    out = out * gate[:, :, None]
    return linear(out.reshape(T, H * vdim), w["o"])


def linear_side(h: torch.Tensor, w: dict, m: dict, eps: float,
                state: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """The gated-linear-attention side, token by token. Returns the output and the state
    after the last token (``[heads, dim, vdim]``); ``state`` continues an earlier stretch."""
    T = h.shape[0]
    H, dim, vdim, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (linear(h, w["q"]) * dim ** -0.5).reshape(T, H, dim)
    k = linear(h, w["k"]).reshape(T, H, dim)
    v = linear(h, w["v"]).reshape(T, H, vdim)
    z = linear(linear(h, w["a1"]), w["a2"], w["a2.b"]).reshape(T, H, dim)
    out, S = decayed_memory(q, k, v, z, tau, state)
    out = rms(out, eps) * w["norm"]  # every head over its own vdim entries, one shared weight
    out = out.reshape(T, H * vdim) * silu(linear(h, w["g"]))
    return linear(out, w["o"]), S


def side_by_side(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Both sides read the same input; each result is normed over the model width with its
    own weight; the mixer returns their mean."""
    left = softmax_side(h, sub(w, "left."), m["left"], eps)
    right, _ = linear_side(h, sub(w, "right."), m["right"], eps)
    return 0.5 * (weighted_norm(left, w["left.out"], eps)
                  + weighted_norm(right, w["right.out"], eps))


# ---------------------------------------------------------------------------------------------
# feed-forward


def expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
           limit: float) -> torch.Tensor:
    g = torch.clamp(linear(h, gate), max=limit)
    u = torch.clamp(linear(h, up), min=-limit, max=limit)
    return linear(g * torch.sigmoid(1.702 * g) * (u + 1.0), down)


def route(h: torch.Tensor, router: torch.Tensor, top: int) -> tuple[torch.Tensor, torch.Tensor]:
    """The ``top`` largest router logits of each row and the softmax over just those."""
    logits = linear(h, router)
    chosen_logits, chosen = torch.topk(logits, top, dim=-1)
    return chosen, torch.softmax(chosen_logits, dim=-1)


def mixture(h: torch.Tensor, w: dict, mlp: dict) -> torch.Tensor:
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    chosen, share = route(h, w["router"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(chosen[t, j])
            out[t] += share[t, j] * expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"],
                                           w[f"e{e}.down"], limit)[0]
    return out


# ---------------------------------------------------------------------------------------------
# the model


def sub(w: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t for name, t in w.items() if name.startswith(prefix)}


def layer(x: torch.Tensor, w: dict, entry: dict, eps: float) -> torch.Tensor:
    if entry["type"] != "parallel":
        raise ValueError(f"unknown layer type {entry['type']!r}")
    h = weighted_norm(x, w["norm1"], eps)
    x = x + w["ls1"] * side_by_side(h, sub(w, "mix."), entry["mixer"], eps)
    if entry.get("mlp") is not None:
        h = weighted_norm(x, w["norm2"], eps)
        x = x + w["ls2"] * mixture(h, sub(w, "mlp."), entry["mlp"])
    return x


def residual_after_layers(state: dict, config: dict, tokens: torch.Tensor) -> list[torch.Tensor]:
    eps = config["norm"]["eps"]
    x = state["embed"][tokens]
    out = []
    for index, entry in enumerate(config["layers"]):
        x = layer(x, sub(state, f"l{index}."), entry, eps)
        out.append(x)
    return out


def logits(state: dict, config: dict, tokens: torch.Tensor) -> torch.Tensor:
    eps = config["norm"]["eps"]
    x = state["embed"][tokens]
    for index, entry in enumerate(config["layers"]):
        x = layer(x, sub(state, f"l{index}."), entry, eps)
    return linear(weighted_norm(x, state["final.norm"], eps), state["head"])


def router_margins(state: dict, config: dict, tokens: torch.Tensor) -> torch.Tensor:
    """Per position, the smallest over the layers of: the gap between the last chosen and the
    first unchosen router logit, as a fraction of the layer's largest logit. Where the margin
    is below the rounding of an engine's arithmetic the model is discontinuous: another
    expert may rightly be chosen there, and the logits jump."""
    eps = config["norm"]["eps"]
    x = state["embed"][tokens]
    margin = torch.full((tokens.shape[0],), float("inf"), dtype=x.dtype)
    for index, entry in enumerate(config["layers"]):
        w = sub(state, f"l{index}.")
        mlp = entry.get("mlp")
        if mlp is not None:
            h = weighted_norm(x, w["norm1"], eps)
            mid = x + w["ls1"] * side_by_side(h, sub(w, "mix."), entry["mixer"], eps)
            z = linear(weighted_norm(mid, w["norm2"], eps), w["mlp.router"])
            top = mlp["router"]["top"]
            if top < z.shape[1]:
                ordered, _ = torch.sort(z, dim=-1, descending=True)
                margin = torch.minimum(margin, (ordered[:, top - 1] - ordered[:, top])
                                       / z.abs().max())
        x = layer(x, w, entry, eps)
    return margin


def cast_state(state: dict, dtype: torch.dtype) -> dict:
    return {name: t.to(dtype) if t.is_floating_point() else t for name, t in state.items()}


def greedy_generate(state: dict, config: dict, prompt: list[int], count: int) -> list[int]:
    """``count`` tokens, each the largest logit (smallest id on ties) of the whole sequence
    so far run from scratch."""
    tokens = list(prompt)
    for _ in range(count):
        last = logits(state, config, torch.tensor(tokens))[-1]
        tokens.append(int(torch.argmax(last)))
    return tokens[len(prompt):]
