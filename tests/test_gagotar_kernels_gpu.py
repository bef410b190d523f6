"""Gagotar's kernels, each alone against the plain formulas in float64: the prepare step and
the attention with mixed heads over scrambled pages, the gated linear attention's scan carried
through cuts, the gated norm with a shared weight, the join of the two sides, routing and the
grouped products of the experts."""

from __future__ import annotations

import pytest
import torch

import plain_gagotar as plain
from ayaka_b200.kernels import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got: torch.Tensor, want: torch.Tensor, dtype: torch.dtype, label: str,
           bf16_limit: float = 2e-2) -> None:
    limit = 2e-5 if dtype == torch.float32 else bf16_limit
    scale = float(want.abs().max())
    error = float((got.double().cpu() - want).abs().max())
    assert error <= limit * scale, f"{label}: {error:.3e} of scale {scale:.3e}"


# ---- prepare + attention -------------------------------------------------------------------
def _attention_case(dtype, *, H, G, dim, vdim, chunk, page, turned, lengths, cut, normed, loud,
                    seed):
    """Requests of ``lengths`` tokens; the first ``cut[b]`` tokens of request b are stored by
    one call of the prepare kernel, the rest are stored and attended by a second step. Pages
    are handed out in a scrambled order and unwritten slots hold NaN."""
    gen = torch.Generator().manual_seed(seed)
    q_w, k_w, v_w = H * dim, G * dim, G * vdim
    ld = q_w + k_w + v_w + H + 3  # the gate follows the values; a few unused columns
    total = sum(lengths)
    proj = torch.randn(total, ld, generator=gen, dtype=torch.float64)
    bias = torch.randn(q_w + k_w + v_w, generator=gen, dtype=torch.float64) * 0.3
    qn = 1 + 0.2 * torch.randn(q_w, generator=gen, dtype=torch.float64)
    kn = 1 + 0.2 * torch.randn(k_w, generator=gen, dtype=torch.float64)
    talk = torch.eye(H, dtype=torch.float64) + 0.4 * torch.randn(H, H, generator=gen,
                                                                 dtype=torch.float64)
    temp = 0.5 + torch.rand(H, generator=gen, dtype=torch.float64)
    scale, eps = 1.5 * dim ** -0.5, 1e-5  # (scores of a few units whatever the head size)
    starts = [sum(lengths[:b]) for b in range(len(lengths))]
    if loud:
        # in every block the first key (the last one a late query still sees) is loud, and
        # the key before it (just outside) louder still; the last query of a block is loud too
        for b, length in enumerate(lengths):
            for t in range(length):
                row = proj[starts[b] + t]
                if t % chunk == 0:
                    row[q_w:q_w + k_w] *= 3.0
                if t % chunk == chunk - 1:
                    row[q_w:q_w + k_w] *= 5.0
                    row[:q_w] *= 2.0
    freq = plain.scaled_frequencies(turned, 40.0, {"factor": 3.0, "low": 1.0, "high": 3.0,
                                                   "original": 30})
    # plain: every request whole
    want = torch.empty(total, H * vdim, dtype=torch.float64)
    for b, length in enumerate(lengths):
        rows = proj[starts[b]:starts[b] + length]
        q = rows[:, :q_w] + bias[:q_w]
        k = rows[:, q_w:q_w + k_w] + bias[q_w:q_w + k_w]
        v = (rows[:, q_w + k_w:q_w + k_w + v_w] + bias[q_w + k_w:]).reshape(length, G, vdim)
        if normed:
            q, k = plain.weighted_norm(q, qn, eps), plain.weighted_norm(k, kn, eps)
        positions = torch.arange(length)
        q = plain.rotate_halves(q.reshape(length, H, dim), positions, freq)
        k = plain.rotate_halves(k.reshape(length, G, dim), positions, freq)
        out = plain.mixed_head_attention(q, k, v, talk, temp, scale, chunk)
        gate = torch.sigmoid(rows[:, q_w + k_w + v_w:q_w + k_w + v_w + H])
        want[starts[b]:starts[b] + length] = (out * gate[:, :, None]).reshape(length, H * vdim)

    # device: pages in a scrambled order
    pages_per = [-(-length // page) for length in lengths]
    num_pages = sum(pages_per) + 3
    order = torch.randperm(num_pages - 1, generator=gen) + 1
    table = torch.zeros(len(lengths), max(pages_per), dtype=torch.int32)
    at = 0
    for b, count in enumerate(pages_per):
        table[b, :count] = order[at:at + count].int()
        at += count
    k_pages = torch.full((num_pages, G, page, dim), float("nan"), dtype=dtype, device=DEV)
    v_pages = torch.full((num_pages, G, page, vdim), float("nan"), dtype=dtype, device=DEV)
    f32 = dict(dtype=torch.float32, device=DEV)
    dev = dict(bias=bias.to(**f32), q_weight=qn.to(**f32) if normed else None,
               k_weight=kn.to(**f32) if normed else None, eps=eps,
               freq=torch.tensor(freq, dtype=torch.float64, device=DEV), layout="halves",
               talk=talk.to(**f32).contiguous(), temp=temp.to(**f32), scale=scale,
               k_pages=k_pages, v_pages=v_pages, heads=H, kv_heads=G, dim=dim, vdim=vdim)
    got = torch.empty(total, H * vdim, dtype=torch.float64)
    for phase in (0, 1):
        spans = [(0, cut[b]) if phase == 0 else (cut[b], lengths[b]) for b in range(len(lengths))]
        rows_of, positions, request_of_row, slots = [], [], [], []
        for b, (lo, hi) in enumerate(spans):
            for t in range(lo, hi):
                rows_of.append(starts[b] + t)
                positions.append(t)
                request_of_row.append(b)
                slots.append(int(table[b, t // page]) * page + t % page)
        n = len(rows_of)
        if n == 0:
            continue
        step_proj = proj[rows_of].to(**f32).contiguous()
        pos = torch.tensor(positions, dtype=torch.int32, device=DEV)
        qmix = torch.empty(n, H * G * dim, dtype=dtype, device=DEV)
        ops.talking_prepare(step_proj, k_offset=q_w, v_offset=q_w + k_w, positions=pos,
                            slot_mapping=torch.tensor(slots, dtype=torch.int32, device=DEV),
                            qmix=qmix, rows=n, **dev)
        if phase == 0:
            continue
        out = torch.full((n, H * vdim), float("nan"), dtype=dtype, device=DEV)
        ops.talking_attention(qmix, k_pages, v_pages, table.to(DEV),
                              torch.tensor(request_of_row, dtype=torch.int32, device=DEV), pos,
                              out, heads=H, chunk=chunk, reach=min(chunk, max(lengths)),
                              gate=step_proj[:, q_w + k_w + v_w:q_w + k_w + v_w + H], rows=n,
                              single_rows=all(hi - lo == 1 for lo, hi in spans))
        torch.cuda.synchronize()
        got[rows_of] = out.double().cpu()
        second = rows_of
    return got[second], want[second]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    dict(H=4, G=2, dim=16, vdim=24, chunk=20, page=16, turned=8, lengths=(61, 20, 3),
         cut=(33, 0, 2)),
    dict(H=3, G=3, dim=8, vdim=4, chunk=5, page=8, turned=8, lengths=(26, 11), cut=(25, 5)),
    dict(H=6, G=1, dim=12, vdim=40, chunk=64, page=16, turned=0, lengths=(150, 64, 65),
         cut=(63, 64, 0)),
    dict(H=1, G=1, dim=32, vdim=32, chunk=300, page=32, turned=32, lengths=(170,), cut=(100,)),
    # sizes of every variant of the tensor-core kernel, more heads than a CTA takes, and
    # steps of single rows (each request's last token alone)
    dict(H=6, G=2, dim=80, vdim=104, chunk=48, page=16, turned=40, lengths=(100, 49, 7),
         cut=(3, 48, 0)),
    dict(H=12, G=4, dim=64, vdim=40, chunk=33, page=16, turned=64, lengths=(70, 34),
         cut=(69, 33)),
    dict(H=2, G=1, dim=64, vdim=72, chunk=16, page=8, turned=2, lengths=(40, 17, 16, 1),
         cut=(39, 16, 15, 0)),
    # steps of single rows: twenty heads (a CTA's sixteen and four more) over five key/value
    # heads, the last key of a block, the first of the next, and a block's only key
    dict(H=20, G=5, dim=16, vdim=16, chunk=50, page=16, turned=8, lengths=(75, 51, 50, 101),
         cut=(74, 50, 49, 100)),
    dict(H=3, G=1, dim=128, vdim=128, chunk=0 + 300, page=16, turned=128, lengths=(290, 17),
         cut=(289, 16)),
    # token-wide keys of 48 entries from heads of 12: the tensor-core kernel without its
    # 16-byte copies, in portions and in single rows
    dict(H=8, G=4, dim=12, vdim=8, chunk=10, page=8, turned=6, lengths=(45, 21), cut=(7, 3)),
    dict(H=8, G=4, dim=12, vdim=8, chunk=10, page=8, turned=6, lengths=(45, 21), cut=(44, 20)),
    # a token's key heads side by side are 512 and 384 entries
    dict(H=4, G=4, dim=128, vdim=128, chunk=40, page=16, turned=64, lengths=(90, 41),
         cut=(10, 40)),
    dict(H=9, G=3, dim=128, vdim=48, chunk=64, page=32, turned=128, lengths=(70,), cut=(5,)),
])
def test_prepare_and_attention_over_scrambled_pages(dtype, case):
    got, want = _attention_case(dtype, normed=True, loud=False, seed=5, **case)
    _close(got, want, dtype, "attention")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_loud_key_just_outside_the_block_is_not_seen(dtype):
    """No norm, so that loud rows stay loud: in every block the first key is loud and the
    key just before it louder still. One position off in the block's start, in prompts or in
    single rows, and the result is another key's value."""
    for cut in ((0, 0), (40, 21), (59, 39), (60 - 1, 41 - 1), (40, 40)):
        # whole; cut inside a block; the last rows; single rows at a block's last and first place
        got, want = _attention_case(dtype, H=4, G=2, dim=8, vdim=8, chunk=20, page=16, turned=4,
                                    lengths=(60, 41), cut=cut, normed=False, loud=True, seed=9)
        # (a fault here moves the result by the size of a value; a score of 20 rounded to
        # eight bits moves a weight by a few per cent)
        _close(got, want, dtype, f"loud edges, cut {cut}", bf16_limit=8e-2)


# ---- the scan --------------------------------------------------------------------------------
@pytest.mark.parametrize("heads,dim,columns", [(3, 5, 7), (2, 24, 20), (1, 40, 16), (2, 100, 12),
                                               (1, 160, 33), (4, 32, 32)])
def test_the_decayed_memory_through_cuts(heads, dim, columns):
    gen = torch.Generator().manual_seed(heads * 100 + dim)
    lengths, tau = (37, 1, 12), 5.0
    qk, inner = heads * dim, heads * columns
    ld = 2 * qk + inner + 5
    total = sum(lengths)
    proj = torch.randn(total, ld, generator=gen, dtype=torch.float64)
    z = 2.0 + 2.0 * torch.randn(total, qk, generator=gen, dtype=torch.float64)
    want = torch.empty(total, inner, dtype=torch.float64)
    last = []
    at = 0
    for length in lengths:
        rows = proj[at:at + length]
        out, S = plain.decayed_memory(
            rows[:, :qk].reshape(length, heads, dim) * dim ** -0.5,
            rows[:, qk:2 * qk].reshape(length, heads, dim),
            rows[:, 2 * qk:2 * qk + inner].reshape(length, heads, columns),
            z[at:at + length].reshape(length, heads, dim), tau)
        want[at:at + length] = out.reshape(length, inner)
        last.append(S)
        at += length
    dproj, dz = proj.float().to(DEV), z.float().to(DEV)
    slots = [4, 0, 2]  # of six: the others must stay as they are
    for cuts in ([1000], [1], [5, 2, 9, 1, 30]):
        state = torch.full((6, heads * dim * columns), 7.0, dtype=torch.float32, device=DEV)
        state[slots] = 0
        got = torch.empty(total, inner, dtype=torch.float32, device=DEV)
        done = [0, 0, 0]
        turn = 0
        while any(done[b] < lengths[b] for b in range(3)):
            rows_of, row_start, live = [], [0], []
            for b in range(3):
                if done[b] == lengths[b]:
                    continue
                size = min(cuts[turn % len(cuts)], lengths[b] - done[b])
                first = sum(lengths[:b]) + done[b]
                rows_of += list(range(first, first + size))
                row_start.append(len(rows_of))
                live.append(b)
                done[b] += size
                turn += 1
            step_proj, step_z = dproj[rows_of].contiguous(), dz[rows_of].contiguous()
            out = torch.empty(len(rows_of), inner, dtype=torch.float32, device=DEV)
            ops.gla_scan(step_proj, step_z, state, out,
                         row_start=torch.tensor(row_start, dtype=torch.int32, device=DEV),
                         state_slot=torch.tensor([slots[b] for b in live], dtype=torch.int32,
                                                 device=DEV),
                         requests=len(live), heads=heads, dim=dim, columns=columns, k_offset=qk,
                         v_offset=2 * qk, tau=tau, q_scale=dim ** -0.5)
            got[rows_of] = out
        _close(got, want, torch.float32, f"scan, cuts {cuts}")
        for b in range(3):  # S is kept as [heads][columns][dim]
            kept = state[slots[b]].view(heads, columns, dim).transpose(1, 2)
            _close(kept, last[b], torch.float32, "state")
        assert bool((state[[1, 3, 5]] == 7.0).all())


# ---- norms and joins -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_gated_norm_with_one_weight_for_every_head(dtype):
    torch.manual_seed(3)
    rows, heads, columns, eps = 9, 5, 12, 1e-5
    x = torch.randn(rows, heads * columns, dtype=torch.float64) * 3
    gate = torch.randn(rows, heads * columns, dtype=torch.float64)
    weight = 1 + 0.3 * torch.randn(columns, dtype=torch.float64)
    want = (plain.rms(x.reshape(rows, heads, columns), eps) * weight).reshape(rows, -1) \
        * plain.silu(gate)
    out = torch.empty(rows, heads * columns, dtype=dtype, device=DEV)
    ops.rms_norm(x.float().to(DEV), weight.float().to(DEV), eps, out, groups=heads,
                 gate=gate.float().to(DEV), gate_mode="silu_after")
    _close(out, want, dtype, "gated norm")


def test_the_join_of_two_sides_and_the_scaled_sum():
    torch.manual_seed(4)
    rows, width, eps = 11, 72, 1e-6
    a, b = torch.randn(rows, width, dtype=torch.float64) * 5, torch.randn(rows, width,
                                                                          dtype=torch.float64)
    wa, wb, scale = (1 + 0.2 * torch.randn(width, dtype=torch.float64) for _ in range(3))
    residual = torch.randn(rows, width, dtype=torch.float64)
    joined = 0.5 * (plain.weighted_norm(a, wa, eps) + plain.weighted_norm(b, wb, eps))
    f32 = dict(dtype=torch.float32, device=DEV)
    dst = residual.to(**f32)
    ops.norm_sum([a.to(**f32), b.to(**f32)], [wa.to(**f32), wb.to(**f32)], eps, dst, factor=0.5,
                 scale=scale.to(**f32), accumulate=True, rows=rows)
    _close(dst, residual + scale * joined, torch.float32, "norm_sum")
    dst = torch.full((rows, width), float("nan"), **f32)
    ops.norm_sum([a.to(**f32)], [wa.to(**f32)], eps, dst, factor=1.0, accumulate=False,
                 rows=rows)
    _close(dst, plain.weighted_norm(a, wa, eps), torch.float32, "norm_sum, one side, written")
    dst = residual.to(**f32)
    ops.scale_add(a.to(**f32), scale.to(**f32), dst, rows=rows)
    _close(dst, residual + scale * a, torch.float32, "scale_add")


# ---- experts ---------------------------------------------------------------------------------
@pytest.mark.parametrize("experts,top", [(5, 2), (3, 1), (40, 40), (70, 3), (1, 1)])
def test_routing(experts, top):
    torch.manual_seed(experts)
    rows = 23
    logits = torch.randn(rows, experts, dtype=torch.float64) * 2
    chosen, share = plain.route(logits, torch.eye(experts, dtype=torch.float64), top)
    got_chosen = torch.empty(rows * top, dtype=torch.int32, device=DEV)
    got_share = torch.empty(rows * top, dtype=torch.float32, device=DEV)
    ops.moe_route(logits.float().to(DEV), got_chosen, got_share, top=top, rows=rows)
    assert got_chosen.view(rows, top).cpu().tolist() == chosen.tolist()
    _close(got_share.view(rows, top), share, torch.float32, "shares")
    assert torch.allclose(got_share.view(rows, top).sum(1).cpu(), torch.ones(rows), atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width,experts,top,ff", [(1, 24, 5, 2, 12), (7, 40, 3, 1, 72),
                                                       (150, 64, 3, 2, 32), (33, 128, 9, 9, 64),
                                                       (700, 72, 4, 2, 80), (90, 36, 2, 1, 44)])
def test_the_experts_against_the_plain_mixture(dtype, rows, width, experts, top, ff):
    """Also more pairs per expert than a tile holds (150 rows, two of three experts each),
    one chosen expert, every expert chosen, the wide tiles of bfloat16 (from 64 pairs per
    expert on), and widths that are no multiple of 8 (no 16-byte pieces)."""
    gen = torch.Generator().manual_seed(rows + experts)
    limit, alpha = 1.2, 1.702

    def draw(*shape, std=1.0):
        return (torch.randn(*shape, generator=gen) * std).to(dtype).double()

    h = draw(rows, width)
    w = {"router": draw(experts, width, std=0.5)}
    for e in range(experts):
        w[f"e{e}.gate"] = draw(ff, width, std=width ** -0.5 * 2)
        w[f"e{e}.up"] = draw(ff, width, std=width ** -0.5 * 2)
        w[f"e{e}.down"] = draw(width, ff, std=ff ** -0.5)
    want = plain.mixture(h, w, {"router": {"top": top}, "expert": {"limit": limit}})
    dev = dict(dtype=dtype, device=DEV)
    w_in = torch.cat([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)])
    w_out = torch.cat([w[f"e{e}.down"] for e in range(experts)])
    logits = (h @ w["router"].T).float().to(DEV)
    chosen = torch.empty(rows * top, dtype=torch.int32, device=DEV)
    share = torch.empty(rows * top, dtype=torch.float32, device=DEV)
    places, tiles = ops.moe_scratch(rows, experts, top)
    pair_out = torch.full((rows * top, width), float("nan"), dtype=torch.float32, device=DEV)
    ops.moe_route(logits, chosen, share, top=top, rows=rows)
    ops.moe_experts(h.to(**dev), w_in.to(**dev).contiguous(), w_out.to(**dev).contiguous(),
                    chosen, pair_out, experts=experts, top=top, limit=limit, alpha=alpha,
                    sorted_pairs=torch.empty(places, dtype=torch.int32, device=DEV),
                    tile_expert=torch.empty(tiles, dtype=torch.int32, device=DEV),
                    inner=torch.empty(places, ff, **dev), rows=rows)
    scale = 1 + 0.1 * torch.randn(width, generator=gen, dtype=torch.float64)
    residual = torch.randn(rows, width, generator=gen, dtype=torch.float64)
    dst = residual.float().to(DEV)
    ops.moe_join(pair_out, share, dst, top=top, scale=scale.float().to(DEV), rows=rows)
    got = dst.double().cpu() - residual
    _close(got, scale * want, dtype, "experts")
