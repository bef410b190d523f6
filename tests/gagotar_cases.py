"""Tiny Gagotar configurations for the tests: each differs from the others in every size and
constant, and none makes equal what a model could happen to make equal (a head's key and
value sizes on either side, the heads of the two sides, the rotated part of a head and the
head, query and key/value heads, chosen experts and one)."""

from __future__ import annotations

import torch

import plain_gagotar as plain
from ayaka_b200.weights.rules import RandomInit

NAME = "Gagotar"


def left(heads, kv_heads, dim, vdim, chunk, *, turned=None, base=10000.0, scale=None,
         scaling=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": scale if scale is not None else dim ** -0.5, "mask": {"size": chunk},
            "rot": {"base": base, "dims": dim if turned is None else turned, "scaling": scaling}}


def right(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top}}


def layer(left_side, right_side, mlp=None):
    return {"type": "parallel", "mixer": {"left": left_side, "right": right_side}, "mlp": mlp}


def model(vocab, width, eps, layers):
    return {"architecture": NAME, "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": layers}


#: wavelengths on both sides of the two thresholds and between them (original 40: a pair
#: with 2 pi / f above 40 is slowed, below 10 kept)
_SCALED = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}

#: two key/value heads for four heads, half of a head rotated with rescaled frequencies, a
#: block of 20 positions (neither a page nor a multiple of one), a layer without feed-forward
TINY_A = model(97, 64, 1e-5, [
    layer(left(4, 2, 16, 24, 20, turned=8, base=300.0, scaling=_SCALED, scale=0.3),
          right(3, 8, 12, 4.0, 5), moe(5, 2, 24, 1.0)),
    layer(left(2, 1, 24, 8, 7, base=50.0), right(1, 24, 8, 9.0, 3)),
    layer(left(4, 2, 16, 24, 20, turned=8, base=300.0, scaling=_SCALED, scale=0.3),
          right(3, 8, 12, 4.0, 5), moe(5, 2, 24, 1.0)),
])

#: as many key/value heads as heads, nothing rotated in one layer, a block shorter than a
#: page and one longer than any test, one expert chosen (its share is one), all experts chosen
TINY_B = model(211, 96, 1e-6, [
    layer(left(3, 3, 8, 16, 5, turned=0), right(2, 12, 20, 2.0, 7), moe(3, 1, 40, 2.5)),
    layer(left(1, 1, 40, 24, 1000, turned=12, base=77.0, scale=0.11), right(5, 4, 8, 30.0, 2),
          moe(4, 4, 16, 0.7)),
])

#: sizes the bfloat16 tensor-core products take (multiples of 8 everywhere); more pairs per
#: expert than a tile of the grouped products holds
TINY_C = model(320, 128, 2e-5, [
    layer(left(4, 1, 32, 16, 48, turned=16, scaling={"factor": 8.0, "low": 1.0, "high": 2.0,
                                                     "original": 16}),
          right(2, 64, 32, 16.0, 8), moe(8, 3, 64, 1.5)),
    layer(left(8, 4, 16, 32, 16), right(4, 16, 48, 6.0, 16), moe(2, 2, 128, 3.0)),
])

#: nothing a multiple of 8 (the CUDA-core products and copies serve bfloat16 too), blocks of
#: three positions and of one (a row sees itself only), a whole-number `original` as a float
TINY_D = model(61, 52, 1e-5, [
    layer(left(5, 5, 6, 10, 3, turned=4, scaling={"factor": 2.0, "low": 1.0, "high": 3.0,
                                                  "original": 12.0}),
          right(2, 5, 7, 3.0, 3), moe(2, 2, 9, 1.1)),
    layer(left(3, 1, 10, 6, 1, base=20.0), right(3, 9, 5, 8.0, 4), moe(7, 3, 11, 2.0)),
])

LOUD = RandomInit(weight_std=0.16, scale_residual_projections=False, bias_std=0.1, norm_std=0.1)
LOUD_WIDE = RandomInit(weight_std=0.1, scale_residual_projections=False, bias_std=0.1,
                       norm_std=0.1)


def plain_logits(state: dict, config: dict, sequences: dict[str, list[int]]
                 ) -> dict[str, torch.Tensor]:
    wide = plain.cast_state(state, torch.float64)
    return {rid: plain.logits(wide, config, torch.tensor(tokens)).float()
            for rid, tokens in sequences.items()}
