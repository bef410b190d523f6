"""A plain, slow Mapuvik: whole sequences, no cache, one function per mechanism, CPU torch.

Mapuvik is a decoder whose layers each pick one of three mixers (a low-rank "latent"
attention with a sliding window, a Mamba-2 state-space layer, an mLSTM matrix memory) and
run it *beside* a dense feed-forward from one shared norm. This file restates the formulas
token by token or as whole-sequence sums and shares no code with ``ayaka_b200``: it reads a
checkpoint-named state dict and the plain dict of ``config.json``.

Every function computes in the dtype of its inputs; tests pass float64 tensors.

Notation: ``x`` the residual stream ``[T, width]``, ``h`` the normed input of a layer,
``t`` a position (from 0), ``H`` heads.
"""

from __future__ import annotations

import math

import torch

# ---------------------------------------------------------------------------------------------
# small pieces


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension (eps under the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the deviation from one: rms(x) * (1 + w)."""
    return rms(x, eps) * (1.0 + weight)


def linear(x: torch.Tensor, weight_out_in: torch.Tensor) -> torch.Tensor:
    """y = W x for every row; W is stored [out, in]; no bias anywhere in this design."""
    return x @ weight_out_in.T


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, dims: int,
                 base: float) -> torch.Tensor:
    """Rotary encoding on the first ``dims`` entries of the last dimension, neighbours
    (2i, 2i+1) forming a pair turned by the angle position * base^(-2i/dims); the rest of
    the vector passes. ``v`` is [T, ..., D]; ``positions`` [T]."""
    out = v.clone()
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=v.dtype)
    angle = positions.to(v.dtype)[:, None] * freq[None, :]  # [T, half]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


# ---------------------------------------------------------------------------------------------
# mixers


def latent_attention(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Attention whose keys and values are up-projections of one small latent row per token.

    q = Wq h, per head [dim plain | rot_dim rotated]; (c_raw | kr) = Wdkv h with
    c = rms(c_raw) * w_c the latent and kr one rotated key piece shared by all heads;
    k_h = Wuk_h c, v_h = Wuv_h c; score(t, s) = scale * (q_plain . k_h + q_rot . kr) over
    t - window < s <= t; softmax; heads joined, times sigmoid(Wg h), then Wo.
    """
    T = h.shape[0]
    H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    window = m["mask"]["size"]
    rot_dims, base = m["rot"]["dims"], m["rot"]["base"]
    pos = torch.arange(T)
    q = linear(h, w["q"]).reshape(T, H, dim + rot)
    q_plain, q_rot = q[..., :dim], rotate_pairs(q[..., dim:], pos, rot_dims, base)
    down = linear(h, w["dkv"])
    c = rms(down[:, :rank], eps) * w["dkv.norm"]
    k_rot = rotate_pairs(down[:, rank:], pos, rot_dims, base)  # [T, rot]
    k_plain = linear(c, w["uk"]).reshape(T, H, dim)
    v = linear(c, w["uv"]).reshape(T, H, vdim)
    scores = torch.einsum("thd,shd->hts", q_plain, k_plain) + \
        torch.einsum("thr,sr->hts", q_rot, k_rot)
    scores = scores * m["scale"]
    delta = pos[:, None] - pos[None, :]  # t - s
    visible = (delta >= 0) & (delta < window)
    scores = scores.masked_fill(~visible[None], float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    joined = torch.einsum("hts,shv->thv", weights, v).reshape(T, H * vdim)
    return linear(joined * torch.sigmoid(linear(h, w["g"])), w["o"])


def causal_conv(u: torch.Tensor, taps_weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """Per channel: out[t] = bias + sum_j w[:, j] * u[t - (taps - 1) + j], zeros before 0."""
    T, taps = u.shape[0], taps_weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], dim=0)
    out = bias.expand(T, -1).clone()
    for j in range(taps):
        out = out + padded[j:j + T] * taps_weight[:, j]
    return out


def mamba2(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """State-space layer, one step at a time. Per head with state S [N, P]:
    S <- exp(-exp(A_log) * dt) S + dt * B x^T ; y = S^T C + D x."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = linear(h, w["in"])
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], \
        proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + w["dt_bias"])  # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)  # [T, H]
    per_group = H // G
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for head in range(H):
        g = head // per_group
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = decay[t, head] * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + w["D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return linear(y, w["o"])


def mlstm(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Matrix memory with exponential gates kept stable by a running maximum that starts
    at zero. Per head: i = cap*tanh(i_raw/cap), f = logsigmoid(cap*tanh(f_raw/cap));
    m_t = max(f + m_prev, i); S <- e^(f+m_prev-m_t) S + e^(i-m_t) k v^T; n likewise with k;
    out = S^T q / (max(|n.q|, e^(-m_t)) + 1e-6)."""
    T = h.shape[0]
    H, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = linear(h, w["q"]).reshape(T, H, dim) * dim ** -0.5
    k = linear(h, w["k"]).reshape(T, H, dim)
    v = linear(h, w["v"]).reshape(T, H, vdim)
    i_gate = cap * torch.tanh((linear(h, w["i"]) + w["i.b"]) / cap)
    f_gate = torch.nn.functional.logsigmoid(cap * torch.tanh((linear(h, w["f"]) + w["f.b"]) / cap))
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for head in range(H):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        n = torch.zeros(dim, dtype=h.dtype)
        m_run = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            m_new = torch.maximum(f_gate[t, head] + m_run, i_gate[t, head])
            keep = torch.exp(f_gate[t, head] + m_run - m_new)
            take = torch.exp(i_gate[t, head] - m_new)
            S = keep * S + take * torch.outer(k[t, head], v[t, head])
            n = keep * n + take * k[t, head]
            m_run = m_new
            denom = torch.maximum((n @ q[t, head]).abs(), torch.exp(-m_run)) + 1e-6
            out[t, head] = (S.T @ q[t, head]) / denom
    out = rms(out, eps).reshape(T, H * vdim) * w["norm"]
    return linear(out * torch.sigmoid(linear(h, w["g"])), w["o"])


MIXERS = {"latent_attention": latent_attention, "mamba2": mamba2, "mlstm": mlstm}


def feed_forward(h: torch.Tensor, w: dict, spec: dict | None) -> torch.Tensor:
    if spec is None:
        return torch.zeros_like(h)
    if spec["kind"] != "dense":
        raise ValueError(spec["kind"])
    return linear(gelu_erf(linear(h, w["up"])), w["down"])


# ---------------------------------------------------------------------------------------------
# the model


def sub(state: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t for name, t in state.items() if name.startswith(prefix)}


def layer_streams(state: dict, config: dict, tokens: torch.Tensor) -> list[torch.Tensor]:
    """The residual stream after every layer run, [T, width] each."""
    eps = config["norm"]["eps"]
    x = state["embed"][tokens]
    seen = []
    for index, layer in enumerate(config["layers"]):
        owner = layer.get("weights_of", index)
        h = offset_norm(x, state[f"l{owner}.norm1"], eps)
        mixed = MIXERS[layer["type"]](h, sub(state, f"l{owner}.mix."), layer["mixer"], eps)
        x = x + (mixed + feed_forward(h, sub(state, f"l{owner}.mlp."), layer.get("mlp")))
        seen.append(x)
    return seen


def logits(state: dict, config: dict, tokens: torch.Tensor) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence."""
    x = layer_streams(state, config, tokens)[-1] if config["layers"] else state["embed"][tokens]
    return linear(offset_norm(x, state["final.norm"], config["norm"]["eps"]), state["head"])


def cast_state(state: dict, dtype: torch.dtype) -> dict:
    return {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in state.items()}


def greedy_generate(state: dict, config: dict, prompt: list[int], count: int) -> list[int]:
    ids = list(prompt)
    for _ in range(count):
        ids.append(int(torch.argmax(logits(state, config, torch.tensor(ids))[-1])))
    return ids[len(prompt):]
