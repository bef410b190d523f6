"""Tiny Mapuvik configurations for the tests: each differs from the others in every size and
constant, and none makes equal what a model could happen to make equal (a head's key,
value and latent sizes, the rotated stretch and the part of it that turns, heads per mixer,
groups of the state-space layer and of its norm)."""

from __future__ import annotations

import torch

import plain_mapuvik as plain
from ayaka_b200.weights.rules import RandomInit

NAME = "Mapuvik"


def latent(heads, dim, rot, vdim, rank, window, *, turned=None, base=10000.0, scale=None):
    return {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank,
        "scale": scale if scale is not None else (dim + rot) ** -0.5,
        "mask": {"size": window}, "rot": {"base": base, "dims": turned or rot}}}


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state,
                                        "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def mlstm(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim,
                                       "gate_cap": cap}}


def layer(entry, ff=None, weights_of=None):
    out = {**entry, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def model(vocab, width, eps, layers):
    return {"architecture": NAME, "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": layers}


_A0 = latent(2, 16, 8, 24, 32, 20)
_A1 = mamba(4, 12, 16, 2, 4, 1)
_A2 = mlstm(3, 16, 20, 10.0)
#: all three mixers, a layer without feed-forward, two layers that borrow their tensors
TINY_A = model(97, 64, 1e-5, [layer(_A0, 96), layer(_A1), layer(_A2, 80),
                              layer(_A0, 96, weights_of=0), layer(_A1, weights_of=1)])

_B0 = mlstm(2, 24, 8, 15.0)
_B1 = latent(3, 8, 16, 16, 24, 7, turned=12, base=500.0, scale=0.31)  # window under a page
_B2 = mamba(2, 40, 8, 1, 2, 4)
_B3 = latent(1, 32, 4, 40, 16, 1000, base=77.0)  # one head, a window longer than any test
#: starts with a recurrent layer; a rotated stretch of which only a part turns; a key row
#: whose size is no multiple of 8
TINY_B = model(211, 96, 1e-6, [layer(_B0, 64), layer(_B1, 72), layer(_B2, 56), layer(_B3),
                               layer(_B0, 64, weights_of=0)])

#: sizes the bfloat16 tensor-core products take (multiples of 8 everywhere)
TINY_C = model(320, 128, 2e-5, [layer(latent(4, 32, 16, 24, 64, 48), 256),
                                layer(mamba(4, 32, 32, 2, 3, 2), 192),
                                layer(mlstm(2, 64, 48, 12.0), 128)])

#: no attention at all: nothing is cached in pages
TINY_STATE_ONLY = model(61, 48, 1e-5, [layer(mamba(3, 8, 4, 3, 3, 3), 40),
                                       layer(mlstm(1, 8, 24, 5.0))])

LOUD = RandomInit(weight_std=0.16, scale_residual_projections=False, bias_std=0.1, norm_std=0.1)
LOUD_WIDE = RandomInit(weight_std=0.1, scale_residual_projections=False, bias_std=0.1,
                       norm_std=0.1)


def plain_logits(state: dict, config: dict, sequences: dict[str, list[int]]
                 ) -> dict[str, torch.Tensor]:
    wide = plain.cast_state(state, torch.float64)
    return {rid: plain.logits(wide, config, torch.tensor(tokens)).float()
            for rid, tokens in sequences.items()}
