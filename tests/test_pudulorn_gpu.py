"""The Pudulorn decoder in the engine against the plain implementation (`plain_pudulorn`): every
mechanism alone, every way of cutting requests into steps, slots and pages used again, planted
weights where random ones would hide a fault, and greedy generation through the entry point."""

import copy
import json
import random

import pytest
import torch

import helpers as H
import plain_pudulorn as P
import pudulorn_helpers as U

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
LENGTHS = {"P": [1, 2, 3, 17, 33, 70, 150], "Q": [2, 5, 31, 64, 65, 200]}


def _requests(name, seed, lengths):
    rng = random.Random(seed)
    vocab = U.CONFIGS[name][0]["vocab"]
    return {f"r{i}": U.clear_ids(U.model_folder(name), rng, n, vocab) for i, n in enumerate(lengths)}


# --------------------------------------------------------------------- mechanisms, one at a time

def _model(name, layers, seed, width=72, vocab=61, eps=1e-5):
    cfg = {"architecture": "Pudulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}
    folder = H.tmp_root() / f"pudulorn-one-{name}"
    U.register(folder, cfg, U.random_tensors(cfg, seed))
    return folder, cfg


ALONE = {
    "attention": [U.attention(4, 2, 16, 24, 20, 8, diff=0.3)],
    "attention_one_key_head_whole_turn": [U.attention(3, 1, 48, 16, 50, 48, diff=0.7, base=300.0, scale=0.3)],
    "attention_odd_sizes": [U.attention(2, 2, 10, 33, 7, 4, diff=0.5)],              # no tensor-core kernel takes these
    "attention_every_head_its_own_keys": [U.attention(3, 3, 32, 32, 64, 16, diff=0.2)],
    "attention_wide_values": [U.attention(2, 1, 64, 256, 33, 32, diff=0.4)],         # two column halves of values
    "attention_block_of_one": [U.attention(2, 2, 16, 16, 1, 16, diff=0.5)],          # every token sees itself only
    "attention_with_dense": [U.attention(4, 4, 32, 64, 40, 32, diff=0.6, mlp=U.dense(100, 0.7))],
    "latent": [U.latent(3, 12, 8, 20, 24, 40, 17, scale=0.2, base=5000.0)],
    "latent_one_head": [U.latent(1, 40, 4, 8, 33, 12, 50, scale=0.1, base=50.0)],
    "latent_many_heads": [U.latent(11, 8, 6, 4, 16, 24, 9, scale=0.4, mlp=U.dense(56, 4.0))],
    "latent_tensor_cores": [U.latent(5, 16, 16, 8, 32, 48, 40, scale=0.2)],
    "latent_two_tiles_of_heads": [U.latent(18, 8, 32, 8, 96, 64, 64, scale=0.15, base=1000.0)],
    "latent_wide": [U.latent(2, 8, 32, 8, 256, 32, 25, scale=0.1)],
    "latent_read_twice": [U.latent(2, 8, 8, 8, 16, 16, 12, scale=0.3), U.latent(3, 4, 8, 12, 16, 8, 30, scale=0.3, kv_from=0),
                          U.latent(1, 16, 8, 4, 16, 8, 5, scale=0.2, kv_from=0)],
    "experts_two_of_five_with_shared": [U.latent(2, 8, 8, 8, 16, 16, 12, mlp=U.moe(5, 2, 24, 1.5, shared=40))],
    "experts_one_of_three": [U.attention(2, 2, 16, 16, 30, 8, mlp=U.moe(3, 1, 32))],
    "experts_all_of_four": [U.attention(2, 1, 16, 16, 30, 8, mlp=U.moe(4, 4, 16, 0.5, shared=16))],
    "experts_many_small": [U.latent(2, 8, 8, 8, 16, 16, 12, mlp=U.moe(33, 3, 8, 2.0))],
    "experts_wide": [U.attention(2, 1, 16, 16, 30, 8, mlp=U.moe(4, 2, 136, 1.0, shared=72))],
    "dense_tight_limit": [U.attention(2, 1, 16, 16, 30, 8, mlp=U.dense(64, 0.05))],
    "no_feed_forward": [U.latent(2, 8, 8, 8, 16, 16, 12), U.attention(2, 1, 16, 16, 30, 8)],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_mechanism_alone(which, dtype):
    folder, cfg = _model(which, ALONE[which], 11)
    rng = random.Random(5)
    requests = {"a": U.clear_ids(folder, rng, 90, cfg["vocab"]), "b": U.clear_ids(folder, rng, 1, cfg["vocab"])}
    steps = H.trace_whole(requests)
    got = H.Replayer(folder, dtype, 16, H.peak_tokens(steps, 16)).run(steps)
    U.check(folder, requests, got, dtype)
    # the same tokens in portions and one by one give the same logits
    steps = H.trace_portions({"a": requests["a"]}, random.Random(1))
    got = H.Replayer(folder, dtype, 16, 96, shuffle_seed=2).run(steps)
    U.check(folder, {"a": requests["a"]}, got, dtype)


def _stream():
    class Ctx:
        stream = torch.cuda.current_stream().cuda_stream
    return Ctx


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,experts,top,hidden,ff", [(70, 5, 2, 64, 24), (3, 3, 1, 40, 16), (300, 8, 3, 128, 72), (1, 4, 4, 32, 8)])
def test_grouped_expert_products(dtype, n, experts, top, hidden, ff):
    """Router, grouping and the two grouped products against one expert at a time."""
    from bare_cuda_4gib_b200.kernels import moe as M
    g = torch.Generator().manual_seed(3)
    ctx = _stream()
    h = torch.randn(n, hidden, generator=g).to(dtype).cuda()
    w_router = (3.0 * torch.randn(experts, hidden, generator=g) / hidden ** 0.5).to(dtype).cuda()
    w_up = (torch.randn(experts, 2 * ff, hidden, generator=g) / hidden ** 0.5).to(dtype).cuda()
    w_down = (torch.randn(experts, hidden, ff, generator=g) / ff ** 0.5).to(dtype).cuda()
    slots = n * top
    ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(n, top, device="cuda")
    M.route(ctx, h, w_router, None, top, 1.5, ids, weights, None, n)
    s = torch.softmax(h.double() @ w_router.double().T, -1)
    want_w, want_ids = torch.sort(s, dim=-1, descending=True, stable=True)
    assert torch.equal(ids.cpu().long().sort(-1).values, want_ids[:, :top].cpu().sort(-1).values)
    assert H.row_error(weights.sort(-1).values, 1.5 * want_w[:, :top].sort(-1).values) < 1e-5
    sorted_slots = torch.empty(slots, dtype=torch.int32, device="cuda")
    tiles = torch.zeros(3 * M.max_tiles(slots, experts) + 1, dtype=torch.int32, device="cuda")
    n_tiles = tiles[3 * M.max_tiles(slots, experts):]
    M.sort(ctx, ids, slots, experts, sorted_slots, tiles, n_tiles)
    order = sorted_slots.cpu().long()
    assert sorted(order.tolist()) == list(range(slots))
    assert (ids.view(-1).cpu()[order].diff() >= 0).all()           # grouped by expert
    act = torch.zeros(slots, ff, dtype=dtype, device="cuda")
    M.grouped(ctx, h, w_up, act, False, sorted_slots, tiles, n_tiles, weights, top, ff, hidden, slots, experts)
    y = torch.zeros(slots, hidden, device="cuda")
    M.grouped(ctx, act, w_down, y, True, sorted_slots, tiles, n_tiles, weights, top, hidden, ff, slots, experts)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    hd, flat_ids, flat_w = h.double(), ids.view(-1).long(), weights.view(-1).double()
    for i, slot in enumerate(order.tolist()):
        e, t = int(flat_ids[slot]), slot // top
        gu = w_up[e].double() @ hd[t]
        a = torch.nn.functional.silu(gu[:ff]) * gu[ff:]
        assert H.row_error(act[i], a) < tol, (i, slot)
        want = flat_w[slot] * (w_down[e].double() @ act[i].double())
        assert H.row_error(y[slot], want) < tol, (i, slot)


@pytest.mark.parametrize("n,experts,top,hidden,ff", [(700, 4, 2, 256, 136), (9, 8, 2, 128, 200), (1, 3, 3, 64, 8),
                                                      (300, 6, 1, 72, 264), (150, 33, 3, 64, 40)])
def test_grouped_expert_products_on_tensor_cores(n, experts, top, hidden, ff):
    """The bfloat16 route: rows put in the list's order, then both grouped products as tiles of 128 rows of one
    expert (several tiles per expert, a last tile of a few rows, widths that fill no whole tile)."""
    from bare_cuda_4gib_b200.kernels import gemm, moe as M
    g = torch.Generator().manual_seed(5)
    ctx = _stream()
    bf = torch.bfloat16
    h = torch.randn(n + 3, hidden + 8, generator=g).to(bf).cuda()[:n, :hidden]      # rows with a stride of their own
    # a router that prefers low experts, so that the groups differ in size and some may stay empty
    ids = (torch.rand(n, experts, generator=g) ** 2).argsort(-1)[:, :top].to(torch.int32).cuda()
    weights = torch.rand(n, top, generator=g).cuda()
    w_up = (torch.randn(experts * 2 * ff, hidden, generator=g) / hidden ** 0.5).to(bf).cuda()
    w_down = (torch.randn(experts * hidden, ff, generator=g) / ff ** 0.5).to(bf).cuda()
    assert M.GroupedPlan.takes(w_up, w_down)
    plan = M.GroupedPlan(w_up, w_down, experts)
    slots = n * top
    sorted_slots = torch.empty(slots, dtype=torch.int32, device="cuda")
    most = M.max_tiles(slots, experts, True)
    tiles = torch.zeros(3 * most + 1, dtype=torch.int32, device="cuda")
    n_tiles = tiles[3 * most:]
    M.sort(ctx, ids, slots, experts, sorted_slots, tiles, n_tiles, True)
    assert int(n_tiles) <= most
    order = sorted_slots.cpu().long()
    rows_in = torch.full((slots + 5, hidden), float("nan"), dtype=bf, device="cuda")[:slots]   # what lies behind is not read into a result
    M.gather_rows(ctx, h, sorted_slots, top, rows_in, slots)
    assert torch.equal(rows_in.cpu(), h.cpu()[order // top])
    act = torch.full((slots, ff), 7.0, dtype=bf, device="cuda")
    y = torch.full((slots, hidden), 7.0, device="cuda")
    M.grouped_tensor(ctx, plan, rows_in, act, False, sorted_slots, tiles, n_tiles, weights, slots)
    M.grouped_tensor(ctx, plan, act, y, True, sorted_slots, tiles, n_tiles, weights, slots)
    gemm.check_errors()
    e_of = ids.view(-1).cpu().long()[order]
    up3, down3 = w_up.double().cpu().view(experts, 2 * ff, hidden), w_down.double().cpu().view(experts, hidden, ff)
    gu = torch.einsum("sfk,sk->sf", up3[e_of], h.double().cpu()[order // top])
    want_act = torch.nn.functional.silu(gu[:, :ff]) * gu[:, ff:]
    rows_error = lambda got, want: float(((got.double().cpu() - want).abs().amax(-1) / want.abs().amax(-1)).max())
    assert rows_error(act, want_act) < 3e-2
    want_y = weights.view(-1).double().cpu()[order, None] * torch.einsum("shf,sf->sh", down3[e_of], act.double().cpu())
    assert rows_error(y.cpu()[order], want_y) < 1e-2


# ------------------------------------------------------------------ every cutting, two configs

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_whole(name, dtype):
    folder, page = U.model_folder(name), U.CONFIGS[name][1]
    requests = _requests(name, 1, LENGTHS[name])
    steps = H.trace_whole(requests)
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page)).run(steps)
    U.check(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_prefill_then_token_by_token(name, dtype):
    folder, page = U.model_folder(name), U.CONFIGS[name][1]
    requests = _requests(name, 2, LENGTHS[name][3:])
    steps = H.trace_decode_tail(requests, 45)          # windows and blocks' edges pass over decoded tokens
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page), shuffle_seed=3).run(steps)
    U.check(folder, requests, got, dtype, expect_all=False)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_portions_down_to_two_tokens(name, dtype):
    folder, page = U.model_folder(name), U.CONFIGS[name][1]
    requests = _requests(name, 3, LENGTHS[name][2:])
    steps = H.trace_portions(requests, random.Random(5))
    got = H.Replayer(folder, dtype, page, H.peak_tokens(steps, page), shuffle_seed=4).run(steps)
    U.check(folder, requests, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_portions_of_two(name, dtype):
    """Every step brings two tokens (the last one perhaps one)."""
    folder, page = U.model_folder(name), U.CONFIGS[name][1]
    ids = _requests(name, 12, [75])["r0"]
    steps = [{"step": i, "entries": [{"id": "r0", "tokens": ids[at: at + 2], "want": list(range(len(ids[at: at + 2])))}], "end": []}
             for i, at in enumerate(range(0, len(ids), 2))]
    got = H.Replayer(folder, dtype, page, 96, shuffle_seed=8).run(steps)
    U.check(folder, {"r0": ids}, got, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_mixed_batches_reuse_slots_and_pages(name, dtype):
    """Unequal requests side by side, four slots and a small pool for eleven requests: every logit
    equals the request's alone, whatever slot and pages it got and whoever held them before."""
    folder, page = U.model_folder(name), U.CONFIGS[name][1]
    longest = 160
    rng = random.Random(11)
    requests = _requests(name, 4, [rng.randrange(3, longest // 2) for _ in range(10)] + [longest])
    budget = 2 * longest
    steps = H.trace_mixed(requests, random.Random(6), live=4, budget_tokens=budget, page=page)
    rep = H.Replayer(folder, dtype, page, budget, max_live=4, shuffle_seed=9)
    got = rep.run(steps)
    U.check(folder, requests, got, dtype)
    for group in rep.cache.groups:
        assert group.pool.acquired_total > group.pool.num_pages and group.pool.pages_in_use == 0
    assert rep.cache.free_slots == 4


@pytest.mark.parametrize("name", ["P", "Q"])
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

def planted(layer, seed, name):
    """One layer whose scores are decided by two tokens.  Token 1's embedding lies along one direction,
    which only the queries read; token 0's along a second one, which only the keys read; every other
    token's is orthogonal to both.  The query of a token 1 and the key of a token 0 are made to
    point the same way (in the first map only, where there are two), so a token 1 finds the earlier
    tokens 0 that it may see, however far back, far above every other key."""
    cfg = {"architecture": "Pudulorn", "vocab": 53, "width": 64, "norm": {"eps": 1e-6}, "layers": [layer]}
    t = {k: v.float() for k, v in U.random_tensors(cfg, seed).items()}
    t["embed"][:, :2] = 0.0
    t["embed"][:2] = 0.0
    t["embed"][1, 0] = 1.0
    t["embed"][0, 1] = 1.0
    t["l0.norm1"][:] = 0.0
    m = layer["mixer"]
    if layer["type"] == "attention":
        d, rot = m["dim"], m["rot"]["dims"]
        way = torch.zeros(d)
        way[rot:] = 1.0                                  # entries that no rotation turns
        q, k = t["l0.mix.q"].view(m["heads"], 2, d, -1), t["l0.mix.k"].view(m["kv_heads"], 2, d, -1)
        q[..., :2], k[..., :2] = 0.0, 0.0
        q[:, 0, :, 0] = way
        k[:, 0, :, 1] = way
        t["l0.mix.q.norm"][:], t["l0.mix.k.norm"][:] = 1.0, 1.0
    else:
        rank, d, r = m["kv_rank"], m["dim"], m["rot_dim"]
        t["l0.mix.dkv"][:, :2] = 0.0
        t["l0.mix.dkv"][:rank, 1] = 2.0
        t["l0.mix.dkv.norm"][:], t["l0.mix.dq.norm"][:] = 1.0, 1.0
        key = t["l0.mix.uk"].sum(1).view(m["heads"], d)            # a head's plain key for an all-ones latent
        t["l0.mix.dq"][:, :2] = 0.0
        t["l0.mix.dq"][:, 0] = 1.0
        uq = t["l0.mix.uq"].view(m["heads"], d + r, -1)
        uq[:, :d, :] += 4.0 * key[:, :, None] / uq.shape[-1]
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    folder = H.tmp_root() / f"pudulorn-planted-{name}"
    U.register(folder, cfg, t)
    return folder, cfg


def moved(folder, cfg, ids, other, at):
    return H.row_error(P.forward(cfg, U._tensors[str(folder)], other)[at], U.plain_logits(folder, ids)[at])


PLANTED_FAR = {"attention": U.attention(2, 1, 64, 32, 400, 16, diff=0.5, scale=0.5),
               "latent": U.latent(2, 32, 16, 16, 64, 48, 350, scale=0.25)}


def far_case(kind):
    folder, cfg = planted(PLANTED_FAR[kind], 21, "far-" + kind)
    rng = random.Random(2)
    filler = lambda n: [rng.randrange(2, cfg["vocab"]) for _ in range(n)]
    ids = filler(9) + [0] + filler(290) + [1] + filler(3)      # the far key is 291 positions back, pages away
    without = list(ids)
    without[9] = 5
    return folder, cfg, ids, without, 300


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", sorted(PLANTED_FAR))
def test_far_key_decides(kind, dtype):
    folder, cfg, ids, without, at = far_case(kind)
    assert moved(folder, cfg, ids, without, at) > 0.1
    requests = {"p": ids}
    got = H.Replayer(folder, dtype, 16, 304).run(H.trace_whole(requests))
    U.check(folder, requests, got, dtype)
    got = H.Replayer(folder, dtype, 16, 304, shuffle_seed=5).run(H.trace_decode_tail(requests, 8))
    U.check(folder, requests, got, dtype, expect_all=False)
    got = H.Replayer(folder, dtype, 16, 304, shuffle_seed=6).run(H.trace_portions(requests, random.Random(3)))
    U.check(folder, requests, got, dtype)


EDGES = [("latent", U.latent(2, 32, 16, 16, 64, 48, 37, scale=0.25), 70, 37),
         ("latent", U.latent(3, 16, 8, 8, 32, 16, 16, scale=0.3), 70, 16),
         ("latent", U.latent(1, 64, 32, 32, 128, 64, 64, scale=0.2), 70, 64),
         # blocks of 50 positions: the planted key opens one, or is the last of the one before
         ("attention", U.attention(2, 1, 64, 32, 50, 16, diff=0.5, scale=0.5), 100, 50),
         ("attention", U.attention(2, 2, 32, 64, 16, 8, diff=0.3, scale=0.7), 64, 16),
         ("attention", U.attention(4, 2, 16, 16, 64, 4, diff=0.7, scale=1.0), 128, 64)]


def edge_case(i):
    kind, layer, start, size = EDGES[i]
    folder, cfg = planted(layer, 23, f"edge{i}")
    rng = random.Random(6)
    filler = lambda n: [rng.randrange(2, cfg["vocab"]) for _ in range(n)]
    # the last position that still sees the planted key at `start`, and the first that does not
    ids = filler(start) + [0] + filler(size - 2) + [1, 1] + filler(5)
    inside, outside = start + size - 1, start + size
    without = list(ids)
    without[start] = 7
    return folder, cfg, ids, without, inside, outside


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("i", range(len(EDGES)))
def test_window_and_block_edges(i, dtype):
    """A planted key just inside the window or block (size - 1 positions back) and just outside (size
    back), in a prompt, in a portion that starts between the two, and for a token decoded alone."""
    folder, cfg, ids, without, inside, outside = edge_case(i)
    assert moved(folder, cfg, ids, without, inside) > 0.05 and moved(folder, cfg, ids, without, outside) < 1e-9
    requests = {"p": ids}
    got = H.Replayer(folder, dtype, 16, 256).run(H.trace_whole(requests))
    U.check(folder, requests, got, dtype)
    cut = inside - 1
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": ids[:cut], "want": [cut - 1]}], "end": []},
             {"step": 1, "entries": [{"id": "p", "tokens": ids[cut: outside + 3], "want": list(range(outside + 3 - cut))}], "end": ["p"]}]
    got = H.Replayer(folder, dtype, 16, 256, shuffle_seed=3).run(steps)
    U.check(folder, requests, got, dtype, expect_all=False)
    got = H.Replayer(folder, dtype, 16, 256, shuffle_seed=4).run(H.trace_decode_tail(requests, 9))
    U.check(folder, requests, got, dtype, expect_all=False)
    assert {("p", inside), ("p", outside)} <= set(got)


@pytest.mark.parametrize("dtype", DTYPES)
def test_borrowed_latent_outlives_the_lenders_window(dtype):
    """The layer that reads another's cached latent looks further back than that layer itself."""
    lender = U.latent(2, 16, 8, 8, 32, 16, 6, scale=0.3)
    reader = U.latent(2, 32, 8, 16, 32, 48, 90, scale=0.25, kv_from=0)
    cfg = {"architecture": "Pudulorn", "vocab": 53, "width": 64, "norm": {"eps": 1e-6}, "layers": [lender, reader]}
    folder = H.tmp_root() / "pudulorn-borrowed"
    U.register(folder, cfg, U.random_tensors(cfg, 9))
    rng = random.Random(7)
    ids = H.random_ids(rng, 140, 53)
    other = list(ids)
    other[60] = (ids[60] + 1) % 53
    assert moved(folder, cfg, ids, other, 139) > 1e-4       # 79 back: only the reader sees it
    got = H.Replayer(folder, dtype, 16, 144, shuffle_seed=2).run(H.trace_decode_tail({"p": ids}, 100))
    U.check(folder, {"p": ids}, got, dtype, expect_all=False)
    got = H.Replayer(folder, dtype, 16, 144, shuffle_seed=3).run(H.trace_portions({"p": ids}, random.Random(4)))
    U.check(folder, {"p": ids}, got, dtype)


# ----------------------------------------------------------------- the entry point and scheduler

@pytest.mark.parametrize("name", ["P", "Q"])
def test_greedy_generation_through_the_engine(name):
    from bare_cuda_4gib_b200.engine.engine import LLMEngine

    folder, page = U.model_folder(name), U.CONFIGS[name][1]
    cfg = U.CONFIGS[name][0]
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
            if token != best:        # a tie within float32 rounding may go either way
                assert float(row[best] - row[token]) < 1e-4 * float(row.abs().max()), (i, token, best)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_layer_by_layer(name):
    """The model cut off after its first layer, its first two, and so on (float32): the first layer
    that differs from the plain implementation is the first cut that fails."""
    cfg, page = U.CONFIGS[name]
    tensors = U.random_tensors(cfg, 3)
    ids = U.clear_ids(U.model_folder(name), random.Random(3), 70, cfg["vocab"])
    for n in range(1, len(cfg["layers"]) + 1):
        cut = dict(cfg, layers=copy.deepcopy(cfg["layers"][:n]))
        kept = {k: v for k, v in tensors.items() if not k.startswith("l") or int(k[1:].split(".")[0]) < n}
        folder = H.tmp_root() / f"pudulorn{name}-first{n}"
        U.register(folder, cut, kept)
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


def test_llm_infer_prints_the_plain_greedy_tokens():
    folder = U.model_folder("Q")
    prompt = [5, 17, 3, 60, 9, 41, 76]
    out = _tool("llm-infer", "--model", folder, "--prompt", ",".join(map(str, prompt)), "--tokens", 10, "--dtype",
                "float32", "--page-tokens", 32)
    generated = [int(t) for t in out.split("generated:")[1].split()]
    assert len(generated) == 10
    logits = U.plain_logits(folder, prompt + generated[:-1])
    assert generated == [int(logits[len(prompt) - 1 + i].argmax()) for i in range(10)]
    assert out.splitlines()[0].startswith("[llm] 5 layers, hidden 96, vocab 77")


def test_tools_run_a_preset_with_random_weights(tmp_path):
    out = _tool("llm-infer", "--model", tmp_path / "m", "--random", "pudulorn-tiny", "--prompt", "1,2,3", "--tokens", 5)
    assert len(out.split("generated:")[1].split()) == 5
    out = _tool("llm-bench", "--model", tmp_path / "m", "--random", "pudulorn-tiny", "--prompt-len", 24, "--tokens", 8,
                "--runs", 2, "--warmup", 1, "--page-tokens", 16)
    assert "TTFT" in out and "TPOT" in out


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_tool(dtype, tmp_path):
    """bin/trace_run on requests that share steps; the third takes the second one's slot and pages."""
    import numpy as np

    folder = U.model_folder("P")
    requests = _requests("P", 17, [40, 19, 33])
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
    vocab = U.CONFIGS["P"][0]["vocab"]
    for step, rows in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), vocab).copy())
        for i, (rid, p) in enumerate(rows):
            err = H.row_error(got[i], U.plain_logits(folder, requests[rid])[p])
            assert err <= U.TOLERANCE[dtype], (step, rid, p, err)
