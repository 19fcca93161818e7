"""The Gurolix decoder in the engine against the plain implementation (`plain_gurolix`): every
mechanism alone, every way of cutting requests into steps, slots and pages used again, planted
weights where random ones would hide a fault, and greedy generation through the entry point."""

import copy
import json
import random

import pytest
import torch

import gurolix_helpers as U
import helpers as H
import plain_gurolix as P

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [1, 2, 3, 17, 33, 70, 150], "B": [2, 5, 31, 64, 65, 200]}
SCALING = (4.0, 1.0, 4.0, 64)


def _requests(name, seed, lengths, dtype="float32"):
    rng = random.Random(seed)
    vocab = U.CONFIGS[name][0]["vocab"]
    return {f"r{i}": U.clear_ids(U.model_folder(name, 3, dtype), rng, n, vocab) for i, n in enumerate(lengths)}


# --------------------------------------------------------------------- mechanisms, one at a time

def _model(name, layers, seed, width=72, vocab=61, eps=1e-5):
    cfg = {"architecture": "Gurolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}
    folder = H.tmp_root() / f"gurolix-one-{name}"
    U.register(folder, cfg, U.random_tensors(cfg, seed))
    return folder, cfg


ALONE = {
    "attention": [U.attention(4, 2, 16, 24, 8)],
    "attention_one_key_head_whole_turn": [U.attention(3, 1, 48, 16, 48, base=300.0, scale=0.3)],
    "attention_odd_sizes": [U.attention(2, 2, 10, 33, 4)],
    "attention_tensor_core_sizes": [U.attention(4, 2, 64, 64, 32)],          # equal heads of 64: the engine's fast kernels
    "attention_wide_values": [U.attention(2, 1, 32, 256, 16)],
    "capped": [U.attention_2(4, 2, 16, 24, 8, 5.0, SCALING, scale=0.5)],
    "capped_tight": [U.attention_2(2, 2, 32, 32, 32, 0.5, (8.0, 1.0, 2.0, 16), base=50.0, scale=1.0)],   # every score near the cap
    "capped_loose_odd": [U.attention_2(6, 3, 12, 20, 6, 1000.0, (2.0, 0.25, 64.0, 1000), scale=0.3)],
    "values_mixed_across_kinds": [U.attention_2(2, 2, 16, 8, 8, 4.0, SCALING, v_mix=True), U.attention(4, 2, 8, 8, 8, v_mix=True),
                                  U.attention(2, 1, 16, 8, 8), U.attention_2(6, 2, 8, 8, 4, 9.0, SCALING, v_mix=True)],
    "mamba2": [U.mamba2(4, 8, 16, 2, 4, 4)],
    "mamba2_one_group_one_tap": [U.mamba2(3, 16, 24, 1, 1, 1)],
    "mamba2_group_per_head_long_taps": [U.mamba2(2, 40, 8, 2, 7, 5)],
    "mamba2_wide_state": [U.mamba2(2, 8, 200, 1, 3, 2)],
    "mamba2_twice": [U.mamba2(2, 16, 16, 2, 2, 1), U.mamba2(4, 8, 8, 1, 4, 2)],
    "mamba2_norm_parts_inside_heads": [U.mamba2(2, 24, 16, 1, 3, 6)],                  # a head spans three parts of the norm
    "mamba2_part_over_two_groups": [U.mamba2(8, 8, 16, 4, 4, 2)],                      # a part's heads read two groups each
    "mamba2_tensor_core_sizes": [U.mamba2(4, 32, 48, 2, 4, 2)],                        # three row tiles of state for four warps
    "mamba2_tensor_core_sizes_wide": [U.mamba2(2, 64, 128, 1, 4, 1)],
    "mamba2_odd_sizes": [U.mamba2(3, 6, 10, 3, 3, 1)],                                # nothing lines up with 16 bytes
    "normed_with_cap_and_rescaled_frequencies": [U.attention(2, 1, 16, 16, 16, scale=0.6)],   # (the options added below)
    "mamba2_wide_heads": [U.mamba2(2, 320, 8, 2, 2, 2)],                               # more value columns than a block has threads
    "experts_with_identity_and_groups": [U.attention(2, 1, 16, 16, 8, mlp=U.moe(5, 2, 24, identity=1, groups=(3, 2)))],
    "experts_mostly_identity": [U.mamba2(2, 8, 8, 1, 2, 1, mlp=U.moe(2, 3, 16, identity=6, groups=(4, 2)))],
    "experts_one_of_three_plain_router": [U.attention(2, 2, 16, 16, 8, mlp=U.moe(3, 1, 32))],
    "experts_all": [U.attention(2, 1, 16, 16, 8, mlp=U.moe(4, 4, 16, groups=(2, 2)))],
    "experts_many_small": [U.mamba2(2, 8, 8, 1, 2, 1, mlp=U.moe(30, 3, 8, identity=3, groups=(11, 4)))],
    "experts_odd_width": [U.attention(2, 1, 16, 16, 8, mlp=U.moe(4, 2, 20, identity=2, groups=(2, 1)))],   # no tile of the tensor-core product fits
    "experts_wide": [U.attention(2, 1, 16, 16, 8, mlp=U.moe(4, 2, 136, identity=2, groups=(3, 2)))],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_mechanism_alone(which, dtype):
    layers = ALONE[which]
    if dtype == "bfloat16":      # routers that choose every expert: see `every_expert_chosen`
        layers = U.every_expert_chosen({"layers": layers})["layers"]
    folder, cfg = _model(f"{which}-{dtype}", layers, 11)
    rng = random.Random(5)
    requests = {"a": U.clear_ids(folder, rng, 90, cfg["vocab"]), "b": U.clear_ids(folder, rng, 1, cfg["vocab"])}
    steps = H.trace_whole(requests)
    got = H.Replayer(folder, dtype, 16, H.peak_tokens(steps, 16)).run(steps)
    U.check(folder, requests, got, dtype)
    # the same tokens in portions and one by one give the same logits
    steps = H.trace_portions({"a": requests["a"]}, random.Random(1))
    got = H.Replayer(folder, dtype, 16, 96, shuffle_seed=2).run(steps)
    U.check(folder, {"a": requests["a"]}, got, dtype)


ALONE["normed_with_cap_and_rescaled_frequencies"][0]["mixer"].update(softcap=3.0)
ALONE["normed_with_cap_and_rescaled_frequencies"][0]["mixer"]["rot"].update(
    scaling=dict(zip(("factor", "low", "high", "original"), SCALING)))


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_width_that_no_fast_kernel_takes(dtype):
    """Width 50: no product, norm or copy in pieces of 16 bytes fits; every part takes its entry-by-entry form."""
    layers = [U.attention_2(2, 1, 16, 16, 8, 4.0, SCALING, scale=0.4, v_mix=True, mlp=U.moe(3, 2, 8, identity=1, groups=(2, 1))),
              U.mamba2(2, 16, 16, 1, 2, 1, mlp=U.moe(2, 1, 12)), U.attention(3, 1, 32, 16, 16, v_mix=True)]
    if dtype == "bfloat16":
        layers = U.every_expert_chosen({"layers": layers})["layers"]
    folder, cfg = _model(f"width50-{dtype}", layers, 17, width=50, vocab=37)
    rng = random.Random(4)
    requests = {"a": U.clear_ids(folder, rng, 70, 37), "b": U.clear_ids(folder, rng, 3, 37)}
    got = H.Replayer(folder, dtype, 16, 96).run(H.trace_whole(requests))
    U.check(folder, requests, got, dtype)
    got = H.Replayer(folder, dtype, 16, 96, shuffle_seed=3).run(H.trace_decode_tail({"a": requests["a"]}, 20))
    U.check(folder, {"a": requests["a"]}, got, dtype, expect_all=False)


def _stream():
    class Ctx:
        stream = torch.cuda.current_stream().cuda_stream
    return Ctx


@pytest.mark.parametrize("n,experts,identity,top,groups,keep", [(70, 5, 1, 2, 3, 2), (9, 10, 5, 3, 5, 2), (300, 3, 0, 1, 1, 1),
                                                                (40, 30, 3, 3, 11, 4), (5, 2, 6, 3, 4, 2)])
def test_router_with_correction_groups_and_identity(n, experts, identity, top, groups, keep):
    from bare_cuda_4gib_b200.kernels import moe as M
    g = torch.Generator().manual_seed(experts)
    total, hidden = experts + identity, 48
    h = torch.randn(n, hidden, generator=g)
    t = {"r.router": 3.0 * torch.randn(total, hidden, generator=g) / hidden ** 0.5, "r.correction": 0.1 * torch.randn(total, generator=g)}
    r = {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}
    margins = []
    want_ids, want_w = P.route({k: v.double() for k, v in t.items()}, "r.", r, h.double(), margins)
    clear = (margins[0] > 1e-5) & (margins[1] > 1e-5)
    ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(n, top, device="cuda")
    M.route(_stream(), h.cuda(), t["r.router"].cuda(), None, top, 1.0, ids, weights, None, n, t["r.correction"].cuda(), groups, keep)
    assert clear.sum() > 0.8 * n
    assert torch.equal(ids.cpu().long()[clear], want_ids[clear])          # in the order of the choice
    assert H.row_error(weights.cpu()[clear], want_w[clear]) < 1e-5


@pytest.mark.parametrize("n,experts,identity,top,hidden,ff", [(700, 4, 2, 2, 256, 136), (9, 8, 3, 2, 128, 200), (1, 3, 1, 3, 64, 8),
                                                              (150, 33, 0, 3, 64, 40)])
def test_ungated_expert_products_plain_and_on_tensor_cores(n, experts, identity, top, hidden, ff):
    """Grouping that leaves identity slots out, rows in the list's order, both grouped products of experts
    W_down relu(W_up h)^2 in plain arithmetic and as tiles of 128 rows, and the sum with the identity slots."""
    from bare_cuda_4gib_b200.kernels import gemm, moe as M
    g = torch.Generator().manual_seed(5)
    ctx, bf = _stream(), torch.bfloat16
    h = torch.randn(n, hidden, generator=g).to(bf).cuda()
    ids = (torch.rand(n, experts + identity, generator=g) ** 2).argsort(-1)[:, :top].to(torch.int32).cuda()
    weights = torch.rand(n, top, generator=g).cuda()
    w_up = (torch.randn(experts * ff, hidden, generator=g) / hidden ** 0.5).to(bf).cuda()
    w_down = (torch.randn(experts * hidden, ff, generator=g) / ff ** 0.5).to(bf).cuda()
    slots = n * top
    flat = ids.view(-1).cpu().long()
    real = flat < experts
    hd, up3, down3 = h.double().cpu(), w_up.double().cpu().view(experts, ff, hidden), w_down.double().cpu().view(experts, hidden, ff)
    want = torch.zeros(n, hidden, dtype=torch.float64)
    for slot in range(slots):
        t, e, w = slot // top, int(flat[slot]), float(weights.view(-1)[slot])
        want[t] += w * (hd[t] if e >= experts else down3[e] @ (torch.relu(up3[e] @ hd[t]) ** 2).to(bf).double())
    for tc in (False, True):
        sorted_slots = torch.full((slots,), -7, dtype=torch.int32, device="cuda")
        most = M.max_tiles(slots, experts, tc)
        tiles = torch.zeros(3 * most + 1, dtype=torch.int32, device="cuda")
        n_tiles = tiles[3 * most:]
        M.sort(ctx, ids, slots, experts, sorted_slots, tiles, n_tiles, tc)
        listed = int(real.sum())
        order = sorted_slots.cpu().long()
        assert sorted(order[:listed].tolist()) == torch.nonzero(real).view(-1).tolist()      # identity slots are listed nowhere
        assert (order[listed:] == 0).all()
        act = torch.full((slots, ff), 7.0, dtype=bf, device="cuda")
        y = torch.full((slots, hidden), 7.0, device="cuda")
        if tc:
            plan = M.GroupedPlan(w_up, w_down, experts, gated=False)
            rows_in = torch.empty(slots, hidden, dtype=bf, device="cuda")
            M.gather_rows(ctx, h, sorted_slots, top, rows_in, slots)
            M.grouped_tensor(ctx, plan, rows_in, act, False, sorted_slots, tiles, n_tiles, weights, slots)
            M.grouped_tensor(ctx, plan, act, y, True, sorted_slots, tiles, n_tiles, weights, slots)
            gemm.check_errors()
        else:
            M.grouped(ctx, h, w_up, act, False, sorted_slots, tiles, n_tiles, weights, top, ff, hidden, slots, experts, False)
            M.grouped(ctx, act, w_down, y, True, sorted_slots, tiles, n_tiles, weights, top, hidden, ff, slots, experts)
        out = torch.empty(n, hidden, device="cuda")
        M.combine(ctx, y, top, None, None, out, n, hidden, ids, weights, experts, h)
        err = float(((out.double().cpu() - want).abs().amax(-1) / want.abs().amax(-1).clamp_min(1e-3)).max())
        assert err < 2e-2, (tc, err)


@pytest.mark.parametrize("rows,width", [(37, 200), (5, 202), (9, 2048), (70, 4096), (3, 6000)])
def test_gated_step_kernel_alone(rows, width):
    """Gate, norm behind the sublayer, add, depth sum and the next norm against plain arithmetic: widths that go
    entry by entry, in pieces of four, and in a wide block for few rows."""
    from bare_cuda_4gib_b200.kernels import gated_sandwich as GS
    from bare_cuda_4gib_b200.kernels.lib import Partials
    g = torch.Generator().manual_seed(2)
    entries = 4
    x = torch.randn(rows, width, generator=g)
    y = torch.randn(3, rows, width, generator=g)
    gate, bias = torch.randn(rows, width, generator=g), torch.randn(width, generator=g)
    post, nxt = 1 + 0.2 * torch.randn(width, generator=g), 1 + 0.2 * torch.randn(width, generator=g)
    mix = torch.randn(entries, generator=g)
    hist = torch.randn(entries, rows, width, generator=g)
    unit = lambda v, eps: v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
    d = torch.float64
    for gate_dtype, out_dtype in ((torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)):
        res, hs = x.clone().cuda(), hist.clone().cuda()
        gt = gate.to(gate_dtype)
        new = x.to(d) + unit(y.to(d).sum(0) * torch.sigmoid(gt.to(d) + bias.to(d)), 1e-5) * post.to(d)
        out = torch.empty(rows, width, dtype=out_dtype, device="cuda")
        delta = GS.GatedDelta(Partials(y.cuda(), 3), gt.cuda(), bias.cuda(), post.cuda(), 1e-5,
                              GS.DepthMix(hs, entries - 1, mix.cuda()))
        GS.step(res, delta, nxt.cuda(), out, 1e-6, rows)
        mixed = (mix[:-1].to(d)[:, None, None] * hist[:-1].to(d)).sum(0) + mix[-1].to(d) * new
        assert H.row_error(hs[entries - 1], new) < 1e-5           # the layer's own result is kept before the sum
        assert torch.equal(hs[: entries - 1].cpu(), hist[: entries - 1])
        assert H.row_error(res, mixed) < 1e-5
        assert H.row_error(out, unit(mixed, 1e-6) * nxt.to(d)) < (1e-5 if out_dtype == torch.float32 else 1e-2)
    # entry 0 alone (the embedding's output is kept, nothing is added or summed), then the norm
    res, hs = x.clone().cuda(), hist.clone().cuda()
    out = torch.empty(rows, width, device="cuda")
    GS.step(res, GS.GatedDelta(None, None, None, None, 0.0, GS.DepthMix(hs, 0, None)), nxt.cuda(), out, 1e-6, rows)
    assert torch.equal(res.cpu(), x) and torch.equal(hs[0].cpu(), x) and torch.equal(hs[1:].cpu(), hist[1:])
    assert H.row_error(out, unit(x.to(d), 1e-6) * nxt.to(d)) < 1e-5
    # only some rows, nothing pending: the norm of the wanted rows, the stream untouched
    res = x.clone().cuda()
    index = torch.tensor([min(5, rows - 1), 0, rows - 1], dtype=torch.int32, device="cuda")
    out = torch.empty(3, width, dtype=torch.bfloat16, device="cuda")
    GS.step(res, None, nxt.cuda(), out, 1e-6, 3, index)
    assert torch.equal(res.cpu(), x)
    assert H.row_error(out, (unit(x.to(d), 1e-6) * nxt.to(d))[index.cpu().long()]) < 1e-2


@pytest.mark.parametrize("heads,vdim,state,groups", [(4, 64, 128, 2), (3, 16, 16, 3), (2, 32, 48, 1), (2, 96, 32, 2)])
def test_chunked_walk_against_the_scan(heads, vdim, state, groups):
    """The recurrence in chunks on the tensor cores against the float32 scan on the same inputs: three requests of
    unequal length (one shorter than a chunk, one that ends inside its fourth), states that are not empty."""
    from bare_cuda_4gib_b200.engine.step import Workspace
    from bare_cuda_4gib_b200.kernels import linear_attention as LA, mamba2 as MK
    g = torch.Generator().manual_seed(heads)
    lengths, taps = [200, 37, 64], 3
    n, inner = sum(lengths), heads * vdim
    C = inner + 2 * groups * state
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")

    class Ctx:
        stream = torch.cuda.current_stream().cuda_stream
        dtype = torch.bfloat16
        n_tokens, n_seqs, max_q_len = n, len(lengths), max(lengths)
        positions = i32([p for q in lengths for p in range(q)])
        row_seq = i32([s for s, q in enumerate(lengths) for _ in range(q)])
        seq_slot = i32([2, 0, 1])
        seq_q_start = i32([0, 200, 237])
        seq_q_len = i32(lengths)
        seq_kv_len = i32(lengths)
        ws = Workspace(torch.device("cuda"), n)

    u = torch.randn(n, inner + C + heads, generator=g).to(torch.bfloat16).cuda()
    conv_w = (torch.randn(C, taps, generator=g) / taps ** 0.5).cuda()
    conv_b = (0.2 * torch.randn(C, generator=g)).cuda()
    ring = torch.zeros(4, taps, C, device="cuda")
    dt_bias, a_log = torch.randn(heads, generator=g).cuda(), (0.5 * torch.randn(heads, generator=g) - 1.0).cuda()
    start = torch.randn(4, heads, state, vdim, generator=g).cuda()
    f32 = dict(dtype=torch.float32, device="cuda")
    qf, kf = torch.empty(n, heads * state, **f32), torch.empty(n, heads * state, **f32)
    vf, xc, decay = torch.empty(n, inner, **f32), torch.empty(n, inner, **f32), torch.empty(n, heads, **f32)
    MK.operands(Ctx, u, conv_w, conv_b, ring, dt_bias, a_log, qf, kf, vf, xc, decay, heads, vdim, state, groups)
    compact = torch.empty(n, C, dtype=torch.bfloat16, device="cuda")
    dt, la = torch.empty(n, heads, **f32), torch.empty(n, heads, **f32)
    xc2 = torch.empty(n, inner, **f32)
    MK.operands(Ctx, u, conv_w, conv_b, ring, dt_bias, a_log, None, None, None, xc2, None, heads, vdim, state, groups, compact, dt, la)
    r = lambda t: t.to(torch.bfloat16).float()
    assert torch.equal(xc2, xc) and torch.equal(compact[:, :inner].float(), r(xc))
    assert torch.allclose(torch.exp(la), decay, rtol=1e-6) and torch.allclose(dt.repeat_interleave(vdim, 1) * xc, vf, rtol=1e-6)
    # the scan on what the chunked walk gets: B, C and x rounded to bfloat16, step sizes and decays as they are
    want_state, want = start.clone(), torch.empty(n, inner, **f32)

    class F32(Ctx):
        dtype = torch.float32
    LA.scan(F32, r(qf), r(kf), dt.repeat_interleave(vdim, 1) * r(xc), decay, "token", want_state, want, heads, state, vdim)
    for columns in (0, 16):      # value columns of a block: the default for the size, and the narrow form
        got_state, got = start.clone(), torch.full((n, inner), float("nan"), **f32)
        MK.chunked(Ctx, compact, dt, la, got_state, got, heads, vdim, state, groups, columns)
        torch.cuda.synchronize()
        assert torch.equal(got_state[3], start[3])                    # a slot that no request of the step holds
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) < 2e-3 * scale, float((got - want).abs().max()) / scale
        assert float((got_state - want_state).abs().max()) < 2e-3 * float(want_state.abs().max())


# ------------------------------------------------------------------ every cutting, two configs

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole(name, dtype):
    folder, page = U.model_folder(name, 3, dtype), U.CONFIGS[name][1]
    requests = _requests(name, 1, LENGTHS[name], dtype)
    steps = H.trace_whole(requests)
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page)).run(steps)
    U.check(folder, requests, got, dtype)


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_in_bfloat16_with_the_routers_as_they_are(name):
    """The configurations' own routers in a bfloat16 run: most rows agree; a row behind a tie that rounding
    decided the other way does not, so this run goes by the share of rows only."""
    folder, page = U.model_folder(name), U.CONFIGS[name][1]
    requests = _requests(name, 1, LENGTHS[name])
    steps = H.trace_whole(requests)
    got = H.Replayer(folder, "bfloat16", page, H.peak_tokens(steps, page)).run(steps)
    errors = sorted(H.row_error(got[(rid, p)], U.plain_logits(folder, ids)[p]) for rid, ids in requests.items() for p in range(len(ids)))
    assert errors[int(0.8 * len(errors))] <= U.TOLERANCE["bfloat16"], errors[-20:]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_prefill_then_token_by_token(name, dtype):
    folder, page = U.model_folder(name, 3, dtype), U.CONFIGS[name][1]
    requests = _requests(name, 2, LENGTHS[name][3:], dtype)
    steps = H.trace_decode_tail(requests, 45)
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page), shuffle_seed=3).run(steps)
    U.check(folder, requests, got, dtype, expect_all=False)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_down_to_two_tokens(name, dtype):
    folder, page = U.model_folder(name, 3, dtype), U.CONFIGS[name][1]
    requests = _requests(name, 3, LENGTHS[name][2:], dtype)
    steps = H.trace_portions(requests, random.Random(5))
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page), shuffle_seed=4).run(steps)
    U.check(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_of_two(name, dtype):
    """Every step brings two tokens (the last one perhaps one): shorter than the convolutions' reach."""
    folder, page = U.model_folder(name, 3, dtype), U.CONFIGS[name][1]
    ids = _requests(name, 12, [75], dtype)["r0"]
    steps = [{"step": i, "entries": [{"id": "r0", "tokens": ids[at: at + 2], "want": list(range(len(ids[at: at + 2])))}], "end": []}
             for i, at in enumerate(range(0, len(ids), 2))]
    got = H.Replayer(folder, dtype, page, 96, shuffle_seed=8).run(steps)
    U.check(folder, {"r0": ids}, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_reuse_slots_and_pages(name, dtype):
    """Unequal requests side by side, four slots and a small pool for eleven requests: every logit
    equals the request's alone, whatever slot and pages it got and whoever held them before (a state
    that was not emptied, or a ring of convolution inputs left by the slot's last owner, shows here)."""
    folder, page = U.model_folder(name, 3, dtype), U.CONFIGS[name][1]
    longest = 160
    rng = random.Random(11)
    requests = _requests(name, 4, [rng.randrange(3, longest // 2) for _ in range(10)] + [longest], dtype)
    budget = 2 * longest
    steps = H.trace_mixed(requests, random.Random(6), live=4, budget_tokens=budget, page=page)
    rep = H.Replayer(folder, dtype, page, budget, max_live=4, shuffle_seed=9)
    got = rep.run(steps)
    U.check(folder, requests, got, dtype)
    for group in rep.cache.groups:
        assert group.pool.acquired_total > group.pool.num_pages and group.pool.pages_in_use == 0
    assert rep.cache.free_slots == 4


@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_in_graphs(name):
    """Three tokens of prompt, then a hundred and more one by one (captured as CUDA graphs after the
    second step), two requests of different age side by side."""
    folder, page = U.model_folder(name), U.CONFIGS[name][1]
    requests = _requests(name, 8, [140, 120])
    a, b = requests["r0"], requests["r1"]
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": a[:3], "want": [2]}], "end": []}]
    for i in range(3, 140):
        entries = [{"id": "r0", "tokens": [a[i]], "want": [0]}]
        j = i - 20
        if j == 0:
            entries.append({"id": "r1", "tokens": b[:1], "want": [0]})
        elif 0 < j < 120:
            entries.append({"id": "r1", "tokens": [b[j]], "want": [0]})
        steps.append({"step": i, "entries": entries, "end": []})
    rep = H.Replayer(folder, "float32", page, 320, max_live=4)
    got = rep.run(steps)
    assert rep.runner._graphs, "no step was replayed from a CUDA graph"
    U.check(folder, requests, got, "float32", expect_all=False)


# ------------------------------------------------------------------------------ planted weights

def planted_attention(layer, seed, name):
    """One attention layer whose scores are decided by two tokens.  Token 1's embedding lies along one
    direction, which only the queries read; token 0's along a second one, which only the keys read;
    every other token's is orthogonal to both.  The query of a token 1 and the key of a token 0 point
    the same way in the entries that no rotation turns, so a token 1 finds the earlier tokens 0,
    however far back, far above every other key (under a cap: at the cap, with all others near zero)."""
    cfg = {"architecture": "Gurolix", "vocab": 53, "width": 64, "norm": {"eps": 1e-6}, "layers": [layer]}
    t = {k: v.float() for k, v in U.random_tensors(cfg, seed).items()}
    t["embed"][:, :2] = 0.0
    t["embed"][:2] = 0.0
    t["embed"][1, 0] = 1.0
    t["embed"][0, 1] = 1.0
    t["embed.norm"][:] = 0.0
    t["l0.norm1"][:] = 0.0
    m = layer["mixer"]
    d, rot = m["dim"], m["rot"]["dims"]
    way = torch.zeros(d)
    way[rot:] = 1.0
    q, k = t["l0.mix.q"].view(m["heads"], d, -1), t["l0.mix.k"].view(m["kv_heads"], d, -1)
    q[..., :2], k[..., :2] = 0.0, 0.0
    q[:, :, 0] = way
    k[:, :, 1] = way
    t["l0.mix.q.b"][:], t["l0.mix.k.b"][:] = 0.0, 0.0
    if layer["type"] == "attention":
        t["l0.mix.q.norm"][:], t["l0.mix.k.norm"][:] = 1.0, 1.0
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    folder = H.tmp_root() / f"gurolix-planted-{name}"
    U.register(folder, cfg, t)
    return folder, cfg


def planted_state(seed, name):
    """One Mamba-2 layer that forgets almost nothing (its decay is exp(-dt e^-9)), so a token hundreds of
    positions back is still in the state that a late token reads."""
    layer = U.mamba2(2, 16, 16, 1, 3, 2)
    cfg = {"architecture": "Gurolix", "vocab": 53, "width": 64, "norm": {"eps": 1e-6}, "layers": [layer]}
    t = {k: v.float() for k, v in U.random_tensors(cfg, seed).items()}
    t["l0.mix.A_log"][:] = -9.0
    # every token but token 0 writes almost nothing: its step size is tiny; token 0's is large
    t["embed"][:, 0] = 0.0
    t["embed"][0] = 0.0
    t["embed"][0, 0] = 8.0
    t["embed.norm"][:] = 0.0
    t["l0.norm1"][:] = 0.0
    w_in = t["l0.mix.in"]
    w_in[-2:, :] = 0.0
    w_in[-2:, 0] = 2.0
    t["l0.mix.dt_bias"][:] = -6.0
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    folder = H.tmp_root() / f"gurolix-planted-{name}"
    U.register(folder, cfg, t)
    return folder, cfg


def moved(folder, cfg, ids, other, at):
    return H.row_error(P.forward(cfg, U._tensors[str(folder)], other)[at], U.plain_logits(folder, ids)[at])


PLANTED_FAR = {"attention": U.attention(2, 1, 64, 32, 16, scale=0.5),
               "capped": U.attention_2(2, 1, 48, 16, 16, 12.0, SCALING, scale=0.02)}      # the planted score lies at the cap, the rest near zero


def far_case(kind):
    if kind == "state":
        folder, cfg = planted_state(21, "far-state")
    else:
        folder, cfg = planted_attention(PLANTED_FAR[kind], 21, "far-" + kind)
    rng = random.Random(2)
    filler = lambda n: [rng.randrange(2, cfg["vocab"]) for _ in range(n)]
    ids = filler(9) + [0] + filler(290) + [1] + filler(3)      # the far token is 291 positions back, pages away
    without = list(ids)
    without[9] = 5
    return folder, cfg, ids, without, 300


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["attention", "capped", "state"])
def test_far_token_decides(kind, dtype):
    folder, cfg, ids, without, at = far_case(kind)
    assert moved(folder, cfg, ids, without, at) > 0.1
    requests = {"p": ids}
    got = H.Replayer(folder, dtype, 16, 304).run(H.trace_whole(requests))
    U.check(folder, requests, got, dtype)
    got = H.Replayer(folder, dtype, 16, 304, shuffle_seed=5).run(H.trace_decode_tail(requests, 8))
    U.check(folder, requests, got, dtype, expect_all=False)
    got = H.Replayer(folder, dtype, 16, 304, shuffle_seed=6).run(H.trace_portions(requests, random.Random(3)))
    U.check(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_every_tap_of_the_convolution(dtype):
    """A convolution of six taps whose every tap matters (equal weights): prompts shorter than its reach,
    portions that end inside it, and single tokens right after a slot's first token."""
    layer = U.mamba2(2, 8, 8, 2, 6, 2)
    cfg = {"architecture": "Gurolix", "vocab": 41, "width": 48, "norm": {"eps": 1e-5}, "layers": [layer]}
    t = U.random_tensors(cfg, 4)
    t["l0.mix.conv"] = torch.full_like(t["l0.mix.conv"], 0.5)
    folder = H.tmp_root() / "gurolix-taps"
    U.register(folder, cfg, t)
    rng = random.Random(9)
    ids = H.random_ids(rng, 23, 41)
    short = {f"s{n}": ids[:n] for n in (1, 2, 3, 5, 6, 7)}
    got = H.Replayer(folder, dtype, 16, 64, max_live=8).run(H.trace_whole(short))
    U.check(folder, short, got, dtype)
    for cut in ([1, 1, 1, 1, 1, 1, 1, 16], [2, 3, 1, 4, 13], [5, 1, 6, 11], [7, 16]):
        steps, at = [], 0
        for i, size in enumerate(cut):
            steps.append({"step": i, "entries": [{"id": "p", "tokens": ids[at: at + size], "want": list(range(size))}], "end": []})
            at += size
        got = H.Replayer(folder, dtype, 16, 32, shuffle_seed=1).run(steps)
        U.check(folder, {"p": ids}, got, dtype)


# ------------------------------------------------------------------------------ the entry point

@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_scheduler(name):
    from bare_cuda_4gib_b200.engine.engine import LLMEngine
    folder, (cfg, page) = U.model_folder(name), U.CONFIGS[name]
    rng = random.Random(13)
    prompts = [H.random_ids(rng, n, cfg["vocab"]) for n in (5, 23, 1, 40, 12, 9)]
    engine = LLMEngine(str(folder), max_tokens=96, max_seqs=4, dtype="float32", page_tokens=page, max_step_tokens=24)
    out = engine.generate_batch(prompts, 24)
    alone = engine.generate(prompts[1], 24)
    assert alone == out[1]
    for prompt, new in zip(prompts, out):
        assert len(new) == 24
        logits = U.plain_logits(folder, prompt + new[:-1])
        for i, token in enumerate(new):
            row = logits[len(prompt) - 1 + i]
            best = int(row.argmax())
            if token != best:        # a tie within float32 rounding, or a router's close call, may go either way
                assert float(row[best] - row[token]) < 1e-3 * float(row.abs().max()), (i, token, best)


@pytest.mark.parametrize("name", ["A", "B"])
def test_layer_by_layer(name):
    """The model cut off after its first layer, its first two, and so on (float32): the first layer
    that differs from the plain implementation is the first cut that fails."""
    cfg, page = U.CONFIGS[name]
    tensors = U.random_tensors(cfg, 3)
    for n in range(1, len(cfg["layers"]) + 1):
        cut = dict(cfg, layers=copy.deepcopy(cfg["layers"][:n]))
        kept = {k: v for k, v in tensors.items() if not k.startswith("l") or int(k[1:].split(".")[0]) < n}
        folder = H.tmp_root() / f"gurolix{name}-first{n}"
        U.register(folder, cut, kept)
        ids = U.clear_ids(folder, random.Random(3), 70, cfg["vocab"])
        got = H.Replayer(folder, "float32", page, 96).run(H.trace_whole({"p": ids}))
        U.check(folder, {"p": ids}, got, "float32")


# ------------------------------------------------------------------------- command line tools

def _tool(tool, *args, feed=None):
    import os
    import pathlib
    import subprocess
    import sys

    root = pathlib.Path(__file__).resolve().parents[1]
    done = subprocess.run([sys.executable, str(root / "bin" / tool), *map(str, args)], input=feed, capture_output=True,
                          text=True, env=dict(os.environ, PYTHONDONTWRITEBYTECODE="1"), timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    return done.stdout


def test_tools_run_a_preset_with_random_weights(tmp_path):
    out = _tool("llm-infer", "--model", tmp_path / "m", "--random", "gurolix-tiny", "--prompt", "1,2,3", "--tokens", 5)
    assert len(out.split("generated:")[1].split()) == 5
    out = _tool("llm-bench", "--model", tmp_path / "m", "--random", "gurolix-tiny", "--prompt-len", 24, "--tokens", 8,
                "--runs", 2, "--warmup", 1, "--page-tokens", 16)
    assert "TTFT" in out and "TPOT" in out


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_tool(dtype, tmp_path):
    """bin/trace_run on requests that share steps; the third takes the second one's slot and pages."""
    import numpy as np

    folder = U.model_folder("A", 3, dtype)
    requests = _requests("A", 17, [40, 19, 33], dtype)
    a, b, c = requests["r0"], requests["r1"], requests["r2"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:2], "want": [1]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [16]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[30:39], "want": []}, {"id": "c", "tokens": c, "want": [32]}], "end": ["c"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[39:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    printed = _tool("trace_run", "--model", folder, "--dtype", dtype, "--out", out, "--max-tokens", 128, "--page-tokens", 16,
                    feed="".join(json.dumps(s) + "\n" for s in steps))
    assert [l for l in printed.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    want = {0: [("r0", 0), ("r0", 29), ("r1", 1)], 1: [("r1", 18)], 2: [("r2", 32)], 3: [("r0", 39)]}
    vocab = U.CONFIGS["A"][0]["vocab"]
    for step, rows in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), vocab).copy())
        for i, (rid, p) in enumerate(rows):
            err = H.row_error(got[i], U.plain_logits(folder, requests[rid])[p])
            assert err <= U.TOLERANCE[dtype], (step, rid, p, err)
